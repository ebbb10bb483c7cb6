// Attention forward in plain fp32 for the score-parity mode: fp32 q, k, v and o, every product, the softmax and
// the weighted sum in fp32, no tensor cores.  It exists so that a model whose dense layers run in fp32 can be
// compared with the reference's fp32 torch path without a 16-bit rounding of q, k and v in between; it is not a
// serving kernel (one warp per query row, keys read straight from global memory).
//
// A warp owns one (sample, head, query): pass 1 gives every lane the keys j = lane, lane + 32, ... — the scaled
// dot products of the visible ones go to the warp's slice of shared memory — then the row maximum and the sum of
// exp2 are reduced across the lanes; pass 2 gives every lane the output dimensions d = lane, lane + 32, ... and
// walks all keys (coalesced reads of the value rows).  Same mask rule as the other kernels: valid prefix,
// always-valid suffix, causal, padded queries returning their own value row, packed batches with separate query
// offsets, or an explicit key-validity map.
#include "attn_common.cuh"
#include "tb200_common.cuh"

namespace tb200 {
void count_launch();

namespace {

constexpr int kWarps = 4;
constexpr int kMaxD = 256;

__global__ void __launch_bounds__(kWarps * 32)
attn_f32_kernel(const AttnArgs a, const int D, const int lk_cap) {
    extern __shared__ float smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    float* qs = smem + warp * (kMaxD + lk_cap);   // the query row, then one score per key
    float* ps = qs + kMaxD;
    const int b = blockIdx.x;
    const int h = blockIdx.y;
    const int r = blockIdx.z * kWarps + warp;     // query index inside the sample

    const bool packed = a.cu_rows != nullptr;
    int lq = a.Lq, lk = a.Lk;
    int64_t row_base = 0, q_base = 0;
    if (packed) {
        row_base = a.cu_rows[b];
        lq = lk = a.cu_rows[b + 1] - static_cast<int32_t>(row_base);
        q_base = row_base;
        if (a.cu_rows_q != nullptr) {
            q_base = a.cu_rows_q[b];
            lq = a.cu_rows_q[b + 1] - static_cast<int32_t>(q_base);
        }
    }
    if (r >= lq) return;
    lk = min(lk, lk_cap);
    const int off = (packed && a.cu_rows_q != nullptr) ? max(lk - lq, 0) : 0;   // position of query 0 among the keys
    const int pos = r + off;
    const int valid_len = (a.seq_len != nullptr && !packed) ? min(max(a.seq_len[b], 0), lk) : lk;
    const int ns_start = packed ? lk : min(a.ns_start, lk);
    const bool causal = a.causal != 0;
    const uint8_t* kvalid = (a.key_valid != nullptr && !packed) ? a.key_valid + static_cast<int64_t>(b) * a.Lk : nullptr;

    const float* qp = static_cast<const float*>(a.q) + (packed ? q_base * a.q_sl : static_cast<int64_t>(b) * a.q_sb) +
                      static_cast<int64_t>(h) * a.q_sh + static_cast<int64_t>(r) * a.q_sl;
    const float* kp = static_cast<const float*>(a.k) + (packed ? row_base * a.k_sl : static_cast<int64_t>(b) * a.k_sb) + static_cast<int64_t>(h) * a.k_sh;
    const float* vp = static_cast<const float*>(a.v) + (packed ? row_base * a.v_sl : static_cast<int64_t>(b) * a.v_sb) + static_cast<int64_t>(h) * a.v_sh;
    float* op = static_cast<float*>(a.o) + (packed ? q_base * a.o_sl : static_cast<int64_t>(b) * a.o_sb) +
                static_cast<int64_t>(h) * a.o_sh + static_cast<int64_t>(r) * a.o_sl;

    // a padded query returns its own value row
    if (a.padded_query_self && !packed && pos < lk) {
        const bool padded_query = kvalid != nullptr ? kvalid[pos] == 0 : (pos >= valid_len && pos < ns_start);
        if (padded_query) {
            for (int d = lane; d < D; d += 32) op[d] = vp[static_cast<int64_t>(pos) * a.v_sl + d];
            return;
        }
    }
    for (int d = lane; d < D; d += 32) qs[d] = qp[d];
    __syncwarp();

    float row_max = -INFINITY;
    for (int j = lane; j < lk; j += 32) {
        const bool seen = kvalid != nullptr ? (kvalid[j] != 0 && (!causal || j <= pos))
                                            : attn_visible(pos, j, valid_len, ns_start, lk, causal);
        float s = -INFINITY;
        if (seen) {
            const float* kr = kp + static_cast<int64_t>(j) * a.k_sl;
            float dot = 0.f;
            for (int d = 0; d < D; ++d) dot = fmaf(qs[d], kr[d], dot);
            s = dot * a.scale_log2;
        }
        ps[j] = s;
        row_max = fmaxf(row_max, s);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) row_max = fmaxf(row_max, __shfl_xor_sync(0xffffffffu, row_max, o));
    if (row_max == -INFINITY) {   // no visible key: zeros
        for (int d = lane; d < D; d += 32) op[d] = 0.f;
        return;
    }
    float sum = 0.f;
    for (int j = lane; j < lk; j += 32) {
        const float p = exp2f(ps[j] - row_max);   // exp2f(-inf) = 0 for hidden keys
        ps[j] = p;
        sum += p;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    __syncwarp();
    const float inv = 1.0f / sum;
    const int last = causal ? min(lk, pos + 1) : lk;   // keys beyond the causal limit carry p = 0
    for (int d = lane; d < D; d += 32) {
        float acc = 0.f;
        for (int j = 0; j < last; ++j) acc = fmaf(ps[j], vp[static_cast<int64_t>(j) * a.v_sl + d], acc);
        op[d] = acc * inv;
    }
}

}  // namespace

// fp32 tensors, head_dim up to 256, at most 8192 keys per sample.
int attn_f32_forward(const AttnArgs& a, int head_dim, int max_lq, int max_lk, cudaStream_t stream) {
    if (head_dim > kMaxD || max_lk > 8192) return TB200_ERR_UNSUPPORTED;
    const int lk_cap = max_lk < 1 ? 1 : max_lk;
    const size_t smem = static_cast<size_t>(kWarps) * (kMaxD + lk_cap) * sizeof(float);
    static bool attr_set[64] = {};
    const DeviceInfo& dev = device_info();
    if (!attr_set[dev.index]) {
        cudaFuncSetAttribute(attn_f32_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(kWarps * (kMaxD + 8192) * sizeof(float)));
        attr_set[dev.index] = true;
    }
    const unsigned row_blocks = static_cast<unsigned>((max_lq + kWarps - 1) / kWarps);
    if (a.H > 65535 || row_blocks > 65535) return TB200_ERR_SHAPE;
    dim3 grid(static_cast<unsigned>(a.B), static_cast<unsigned>(a.H), row_blocks);
    attn_f32_kernel<<<grid, kWarps * 32, smem, stream>>>(a, head_dim, lk_cap);
    count_launch();
    return launch_status();
}

}  // namespace tb200
