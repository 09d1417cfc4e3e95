#define NCN_NC 32
#define NCN_BWD
#include "feat_inst.cuh"
