// Activation codes shared by the GEMM epilogues and the elementwise kernels.
#pragma once
#define NB_ACT_NONE 0
#define NB_ACT_RELU 1
#define NB_ACT_TANH 2
#define NB_ACT_GELU 3   // tanh approximation
#define NB_ACT_SILU 4
#define NB_ACT_SIGMOID 5
// `dact` slot only: the aux tensor is ADDED to the result (residual connection fused into the epilogue)
#define NB_AUX_ADD 16

// Split-K workspace: the first NB_GEMM_WS_COUNTERS u32 are per-tile arrival counters (zero at rest),
// fp32 partial tiles follow.
#define NB_GEMM_WS_COUNTERS 1024
