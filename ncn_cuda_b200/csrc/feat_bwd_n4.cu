#define NCN_NC 4
#define NCN_BWD
#include "feat_inst.cuh"
