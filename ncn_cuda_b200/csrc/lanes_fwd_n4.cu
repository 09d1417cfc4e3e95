#define NCN_NG 4
#include "lanes_inst.cuh"
