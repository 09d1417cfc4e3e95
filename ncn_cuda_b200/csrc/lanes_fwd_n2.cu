#define NCN_NG 2
#include "lanes_inst.cuh"
