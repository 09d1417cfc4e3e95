#define NCN_NG 8
#include "pairs_inst.cuh"
