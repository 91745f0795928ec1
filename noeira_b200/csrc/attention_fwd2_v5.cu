// experiment variant of attention_fwd2_tcgen05.cu
#define FA2_VARIANT _v5
#define FA2_SPLIT_P 1
#define FA2_DEC "72"
#define FA2_INC "216"
#define FA2_DEC_N 72
#define FA2_INC_N 216
#include "attention_fwd2_tcgen05.cu"
