#define NCN_NG 8
#define NCN_BWD 1
#include "lanes_inst.cuh"
