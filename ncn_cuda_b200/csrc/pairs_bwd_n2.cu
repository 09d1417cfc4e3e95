#define NCN_NG 2
#define NCN_BWD 1
#include "pairs_inst.cuh"
