// libtornado_b200.so is compiled as ONE translation unit: the kernels share a
// device-side status word and a handful of inline helpers, and a single nvcc
// invocation keeps the build recipe to one line (see tornadovm_b200/build.py).
#include "api.cu"
#include "gemv_f32.cu"
#include "gemv_quant.cu"
#include "gemv_mma.cu"
#include "sgemm.cu"
#include "hgemm.cu"
#include "gemv_static.cu"
#include "peer.cu"
