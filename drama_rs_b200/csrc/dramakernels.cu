// libdramakernels: the B200 (sm_100a) replacement for the MoE / dense-GEMV part of the reference's
// kernel archive. One translation unit; every exported symbol is declared in include/dramakernels.h.
#include "common.cuh"
#include "runtime.cuh"
#include "gemv.cuh"
#include "router.cuh"
#include "moe_decode.cuh"
#include "moe_decode_static.cuh"
#include "moe_decode_fp8.cuh"
#include "moe_prefill_mma.cuh"
#include "moe_prefill_tma.cuh"
#include "moe_prefill_fp8.cuh"
#include "moe_prefill.cuh"
#include "stack_decode.cuh"
#include "quant.cuh"

