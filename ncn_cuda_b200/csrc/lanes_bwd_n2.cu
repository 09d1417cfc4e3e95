#define NCN_NG 2
#define NCN_BWD 1
#include "lanes_inst.cuh"
