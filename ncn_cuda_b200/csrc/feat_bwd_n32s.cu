#define NCN_NC 32
#define NCN_BWD
#define NCN_SAVED
#include "feat_inst.cuh"
