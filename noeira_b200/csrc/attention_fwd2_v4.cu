// experiment variant of attention_fwd2_tcgen05.cu
#define FA2_VARIANT _v4
#define FA2_SPLIT_P 0
#define FA2_DEC "88"
#define FA2_INC "208"
#define FA2_DEC_N 88
#define FA2_INC_N 208
#include "attention_fwd2_tcgen05.cu"
