#define NCN_NC 8
#include "feat_inst.cuh"
