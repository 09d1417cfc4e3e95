#define NCN_NG 16
#include "rows_inst.cuh"
