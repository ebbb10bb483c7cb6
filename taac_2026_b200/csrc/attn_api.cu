// C-ABI entry of the attention forward: argument checks and kernel selection.
#include "attn_common.cuh"
#include "tb200_common.cuh"

namespace tb200 {
int attn_mma_forward(const AttnArgs& a, int head_dim, int dtype, int max_lq, cudaStream_t stream);
bool attn_tc05_supported(const AttnArgs& a, int head_dim, int dtype);
int attn_tc05_forward(const AttnArgs& a, int max_lq, int64_t total_rows, int32_t* status, cudaStream_t stream);
bool attn_small_supported(const AttnArgs& a, int head_dim, int max_lq, int max_lk);
bool attn_tiny_supported(const AttnArgs& a, int head_dim, int max_lq, int max_lk);
bool attn_fewq_supported(const AttnArgs& a, int head_dim);
int attn_fewq_forward(const AttnArgs& a, int dtype, cudaStream_t stream);
int attn_tiny_forward(const AttnArgs& a, int dtype, cudaStream_t stream);
int attn_small_forward(const AttnArgs& a, int dtype, cudaStream_t stream);
int attn_f32_forward(const AttnArgs& a, int head_dim, int max_lq, int max_lk, cudaStream_t stream);
}  // namespace tb200

extern "C" int tb200_attn_fwd(const void* q, const void* k, const void* v, void* o, int32_t B, int32_t H, int32_t Lq,
                              int32_t Lk, int32_t D, const int64_t* strides, const int32_t* seq_len,
                              const int32_t* cu_rows, const int32_t* cu_rows_q, const uint8_t* key_valid, int32_t ns_start, int32_t causal, int32_t padded_query_self,
                              float scale, int dtype, int32_t kernel, int64_t total_rows, int32_t* status_word,
                              void* stream) {
    using namespace tb200;
    if (B < 0 || H < 1 || Lq < 0 || Lk < 0 || D < 1) return TB200_ERR_SHAPE;
    if (B == 0 || Lq == 0) return TB200_OK;
    if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || strides == nullptr) return TB200_ERR_NULL;
    if (dtype != TB200_BF16 && dtype != TB200_F16 && dtype != TB200_F32) return TB200_ERR_DTYPE;
    if (dtype == TB200_F32 ? (D > 256 || D % 4 != 0) : (D != 32 && D != 64 && D != 128)) return TB200_ERR_UNSUPPORTED;
    if (padded_query_self && cu_rows == nullptr && Lq != Lk) return TB200_ERR_SHAPE;
    if (cu_rows_q != nullptr && (cu_rows == nullptr || key_valid != nullptr)) return TB200_ERR_UNSUPPORTED;
    if (ns_start < 0) return TB200_ERR_SHAPE;
    if (!aligned16(q) || !aligned16(k) || !aligned16(v) || !aligned16(o)) return TB200_ERR_ALIGN;
    for (int i = 0; i < 12; ++i)
        if (strides[i] % (dtype == TB200_F32 ? 4 : 8) != 0) return TB200_ERR_ALIGN;  // every row must start on a 16-byte boundary
    if (!device_info().valid) return TB200_ERR_DEVICE;
    AttnArgs a{};
    a.q = q; a.k = k; a.v = v; a.o = o;
    a.q_sb = strides[0]; a.q_sh = strides[1]; a.q_sl = strides[2];
    a.k_sb = strides[3]; a.k_sh = strides[4]; a.k_sl = strides[5];
    a.v_sb = strides[6]; a.v_sh = strides[7]; a.v_sl = strides[8];
    a.o_sb = strides[9]; a.o_sh = strides[10]; a.o_sl = strides[11];
    a.seq_len = seq_len;
    a.cu_rows = cu_rows;
    a.cu_rows_q = cu_rows_q;
    a.key_valid = key_valid;
    a.B = B; a.H = H; a.Lq = Lq; a.Lk = Lk;
    a.ns_start = ns_start > Lk ? Lk : ns_start;
    a.causal = causal != 0;
    a.padded_query_self = padded_query_self != 0;
    a.scale_log2 = scale * 1.4426950408889634f;
    if (cu_rows != nullptr && total_rows < 0) return TB200_ERR_SHAPE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // fp32 tensors: the plain fp32 kernel of the score-parity mode, whatever `kernel` says
    if (dtype == TB200_F32) return attn_f32_forward(a, D, Lq, Lk, s);
    // kernel: 0 = automatic, 1 = mma.sync kernel, 2 = tcgen05 kernel, 3 = one-warp-per-(sample, head) kernel for
    // samples of at most 32 rows, 4 = one-warp-per-(sample, head) kernel for few queries against many keys
    const bool tc_ok = attn_tc05_supported(a, D, dtype) && (cu_rows == nullptr || total_rows > 0);
    if (kernel == 2 && !tc_ok) return TB200_ERR_UNSUPPORTED;
    if (kernel < 0 || kernel > 4) return TB200_ERR_UNSUPPORTED;
    const bool fewq_ok = attn_fewq_supported(a, D);
    if (kernel == 4) return fewq_ok ? attn_fewq_forward(a, dtype, s) : TB200_ERR_UNSUPPORTED;
    const bool small_ok = attn_small_supported(a, D, Lq, Lk);
    if (kernel == 3 && !small_ok) return TB200_ERR_UNSUPPORTED;
    if (cu_rows_q != nullptr) {
        // separate query rows: the scalar kernel up to 32 rows; beyond that the queries are by construction the few
        // rows a caller kept of long samples, which is the streaming kernel's case (the mma.sync kernel on request)
        if (kernel == 2) return TB200_ERR_UNSUPPORTED;
        if (kernel == 3 || (kernel == 0 && small_ok)) return attn_small_forward(a, dtype, s);
        if (kernel == 0 && fewq_ok) return attn_fewq_forward(a, dtype, s);
        return attn_mma_forward(a, D, dtype, Lq, s);
    }
    // samples of at most 32 rows (the non-sequence tokens alone, late in the pyramid): no tensor-core tile pays
    if (kernel == 3 || (kernel == 0 && small_ok)) {
        // up to 16 rows the whole sample is one tensor-core tile per head; 17..32 rows take the scalar kernel
        if (attn_tiny_supported(a, D, Lq, Lk)) return attn_tiny_forward(a, dtype, s);
        return attn_small_forward(a, dtype, s);
    }
    // Automatic choice: the tcgen05 kernel wherever it applies (bf16, head_dim 64, no key_valid map); measured
    // on full-length rows it leads the mma.sync kernel from 128 keys up, causal or not.  Samples shorter than
    // one 128-row block leave most of its tile idle, so those stay on the 64-row mma.sync tiles.
    if (kernel == 2 || (kernel == 0 && tc_ok && Lq >= 128))
        return attn_tc05_forward(a, Lq, total_rows, status_word, s);
    return attn_mma_forward(a, D, dtype, Lq, s);
}
