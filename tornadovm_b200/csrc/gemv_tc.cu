#define TB200_OP_CLASS TB200_PREPARE_GEMV_QUANT
#include "gemv_common.cuh"

TB200_TU_STATUS(gemv_tc)
