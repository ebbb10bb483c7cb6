// Argument block and mask rule shared by the attention kernels.
#pragma once
#include <stdint.h>

namespace tb200 {

// Tensors are addressed as base + b * stride_b + h * stride_h + l * stride_l (+ d), strides in
// elements, head dim contiguous.  With cu_rows != nullptr the batch is PACKED: sample b owns rows
// [cu_rows[b], cu_rows[b+1]) of a [total_rows, H, D]-like tensor (stride_b unused), every one of
// its keys is valid, and Lq = Lk = cu_rows[b+1] - cu_rows[b].
struct AttnArgs {
    const void* q;
    const void* k;
    const void* v;
    void* o;
    int64_t q_sb, q_sh, q_sl;
    int64_t k_sb, k_sh, k_sl;
    int64_t v_sb, v_sh, v_sl;
    int64_t o_sb, o_sh, o_sl;
    const int32_t* seq_len;  // [B] valid-prefix length of the key axis, or nullptr = all valid
    const int32_t* cu_rows;  // [B + 1] or nullptr
    // [B + 1] or nullptr.  Packed batches only: q and o are packed by their own offsets (sample b has
    // cu_rows_q[b+1] - cu_rows_q[b] queries, the LAST rows of its cu_rows[b+1] - cu_rows[b] keys), and the
    // causal rule is aligned at the end: query j of lq sees keys <= j + (lk - lq).
    const int32_t* cu_rows_q;
    const uint8_t* key_valid;  // [B, Lk] bytes (0 = padding) or nullptr; replaces seq_len / ns_start when given
    int32_t B, H, Lq, Lk;
    int32_t ns_start;           // keys >= ns_start are always valid (Lk = no such suffix)
    int32_t causal;             // key <= query (top-left aligned)
    int32_t padded_query_self;  // queries in [seq_len, ns_start) return their own value row
    float scale_log2;           // softmax scale * log2(e)
};

// key c visible to query r?
__device__ __forceinline__ bool attn_visible(int r, int c, int valid_len, int ns_start, int lk, bool causal) {
    return (c < valid_len || c >= ns_start) && c < lk && (!causal || c <= r);
}

}  // namespace tb200
