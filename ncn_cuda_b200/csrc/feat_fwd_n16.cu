#define NCN_NC 16
#include "feat_inst.cuh"
