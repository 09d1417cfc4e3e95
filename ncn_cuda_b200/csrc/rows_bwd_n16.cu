#define NCN_NG 16
#define NCN_BWD 1
#include "rows_inst.cuh"
