#define NCN_NG 4
#define NCN_BWD 1
#include "lanes_inst.cuh"
