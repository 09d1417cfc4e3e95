#define NCN_NG 4
#include "pairs_inst.cuh"
