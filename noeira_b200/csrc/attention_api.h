// Mask modes of the attention kernels.
#pragma once
#define NB_MASK_NONE 0
#define NB_MASK_CAUSAL 1        // k <= q + causal_off
#define NB_MASK_BLOCK_CAUSAL 2  // (k / frame) <= (q / frame)
