#define NCN_NG 8
#include "lanes_inst.cuh"
