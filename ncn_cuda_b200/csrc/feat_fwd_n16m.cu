#define NCN_NC 16
#define NCN_MID
#include "feat_inst.cuh"
