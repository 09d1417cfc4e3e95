#define NCN_NG 2
#include "rows_inst.cuh"
