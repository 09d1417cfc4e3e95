#define NCN_NG 2
#include "pairs_inst.cuh"
