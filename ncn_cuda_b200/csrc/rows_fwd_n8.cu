#define NCN_NG 8
#include "rows_inst.cuh"
