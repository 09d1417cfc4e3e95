#define NCN_NC 2
#include "feat_inst.cuh"
