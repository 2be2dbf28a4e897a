// Single translation unit of libbdattn.so: the kernels share one per-device
// status word, so they are compiled together.
#include "tc05.cuh"
#include "sdpa_tc05.cu"
#include "sdpa_general.cu"
#include "norm_rope.cu"
#include "linear_attn.cu"
#include "rope_tables.cu"
#include "gemm_tc05.cu"
#include "gemm_wide.cu"
#include "elementwise.cu"
#include "attn_map.cu"
#include "capi.cu"
#include "qkvo_static.cu"
