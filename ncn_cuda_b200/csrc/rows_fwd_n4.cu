#define NCN_NG 4
#include "rows_inst.cuh"
