#define NCN_NC 2
#define NCN_BWD
#include "feat_inst.cuh"
