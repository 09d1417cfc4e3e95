#define NCN_NC 32
#include "feat_inst.cuh"
