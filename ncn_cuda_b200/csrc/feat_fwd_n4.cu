#define NCN_NC 4
#include "feat_inst.cuh"
