#define NCN_NC 16
#define NCN_BWD
#include "feat_inst.cuh"
