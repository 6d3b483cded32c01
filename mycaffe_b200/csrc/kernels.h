// Internal alias: the kernels implement exactly the raw entry points of the public header.
#pragma once
#include "mycaffe_attn.h"

// Internal: turn the public (bits, bits_t, mask_mode) triple into the kernels' view; *view stays null for no mask.
struct McaMaskBits;
int mca_mask_bits_view(const uint32_t* bits, const uint32_t* bits_t, int mask_mode, int T, int need_transpose, McaMaskBits* out,
                       const McaMaskBits** view);

// Internal: mca_classify_causal_mask in one launch.  scratch: two device ints that are zero before the call and zero
// again after it (a mismatch count and a ticket; the last block to finish writes *flag).
int mca_classify_causal_mask_ws(const float* mask, int T, int* flag, int* scratch, void* stream);
