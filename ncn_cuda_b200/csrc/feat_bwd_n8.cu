#define NCN_NC 8
#define NCN_BWD
#include "feat_inst.cuh"
