#define NCN_NG 8
#define NCN_BWD 1
#include "pairs_inst.cuh"
