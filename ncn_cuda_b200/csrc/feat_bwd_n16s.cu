#define NCN_NC 16
#define NCN_BWD
#define NCN_SAVED
#include "feat_inst.cuh"
