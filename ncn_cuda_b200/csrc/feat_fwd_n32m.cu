#define NCN_NC 32
#define NCN_MID
#include "feat_inst.cuh"
