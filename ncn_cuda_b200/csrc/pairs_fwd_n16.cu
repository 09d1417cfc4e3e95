#define NCN_NG 16
#include "pairs_inst.cuh"
