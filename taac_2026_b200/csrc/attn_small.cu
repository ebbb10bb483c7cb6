// Attention forward for very short samples (at most 32 queries and 32 keys, head_dim 64): one warp per
// (sample, head); P = 1, 2 or 4 lanes share a query row (each holds 64 / P of its dimensions), so that a
// sample of 9 rows still keeps 18 of the 32 lanes busy.
//
// After the pyramid has dropped the behaviour sequence, a sample of the packed batch is only its handful of
// non-sequence tokens; a 64 x 64 tensor-core tile per (sample, head) is then almost all padding and the launch
// is bound by CTA turnover.  Here the keys and values of a (sample, head) sit in 8 KB of the warp's shared
// memory, every lane keeps its query row and fp32 output row in registers and walks the visible keys with an
// online softmax in fp32.  Shared-memory reads of a key are warp-wide broadcasts.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "attn_common.cuh"
#include "tb200_common.cuh"

namespace tb200 {
void count_launch();

namespace {

constexpr int kD = 64;
constexpr int kMaxL = 32;
constexpr int kWarps = 4;
constexpr int kChunks = kD / 8;   // 16-byte pieces per row

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src) {
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(smem_dst));
    asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(gmem_src) : "memory");
}

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <typename T, int P>
__global__ void __launch_bounds__(kWarps * 32)
attn_small_kernel(const AttnArgs a) {
    constexpr int CPL = kChunks / P;      // 16-byte pieces of a row per lane
    constexpr int kRows = kMaxL / P;      // rows one warp can serve
    __shared__ uint4 kv_s[kWarps][2][kMaxL * kChunks];   // per warp: K rows, V rows
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int64_t pair = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
    if (pair >= static_cast<int64_t>(a.B) * a.H) return;
    const int b = static_cast<int>(pair / a.H);
    const int h = static_cast<int>(pair - static_cast<int64_t>(b) * a.H);

    const bool packed = a.cu_rows != nullptr;
    int lq = a.Lq, lk = a.Lk;
    int64_t row_base = 0, q_base = 0;
    if (packed) {
        row_base = a.cu_rows[b];
        lq = lk = a.cu_rows[b + 1] - static_cast<int32_t>(row_base);
        q_base = row_base;
        if (a.cu_rows_q != nullptr) {   // q and o hold the sample's last lq rows only, packed by their own offsets
            q_base = a.cu_rows_q[b];
            lq = a.cu_rows_q[b + 1] - static_cast<int32_t>(q_base);
        }
    }
    lq = min(lq, kRows);
    lk = min(lk, kMaxL);
    const int off = (packed && a.cu_rows_q != nullptr) ? max(lk - lq, 0) : 0;   // position of query 0 among the keys
    const int valid_len = (a.seq_len != nullptr && !packed) ? min(max(a.seq_len[b], 0), lk) : lk;
    const int ns_start = packed ? lk : min(a.ns_start, lk);
    const bool causal = a.causal != 0;

    const T* qp = static_cast<const T*>(a.q) + (packed ? q_base * a.q_sl : static_cast<int64_t>(b) * a.q_sb) + static_cast<int64_t>(h) * a.q_sh;
    const T* kp = static_cast<const T*>(a.k) + (packed ? row_base * a.k_sl : static_cast<int64_t>(b) * a.k_sb) + static_cast<int64_t>(h) * a.k_sh;
    const T* vp = static_cast<const T*>(a.v) + (packed ? row_base * a.v_sl : static_cast<int64_t>(b) * a.v_sb) + static_cast<int64_t>(h) * a.v_sh;
    T* op = static_cast<T*>(a.o) + (packed ? q_base * a.o_sl : static_cast<int64_t>(b) * a.o_sb) + static_cast<int64_t>(h) * a.o_sh;

    // stage K and V with asynchronous 16-byte copies (piece lane % 8 of rows lane / 8, lane / 8 + 4, ...): all of
    // them are in flight together with the load of the query row, instead of one round trip per four rows
    uint4* ks = kv_s[warp][0];
    uint4* vs = kv_s[warp][1];
    for (int r = lane >> 3; r < lk; r += 4) {
        const int c = lane & 7;
        cp_async16(&ks[r * kChunks + c], reinterpret_cast<const uint4*>(kp + static_cast<int64_t>(r) * a.k_sl) + c);
        cp_async16(&vs[r * kChunks + c], reinterpret_cast<const uint4*>(vp + static_cast<int64_t>(r) * a.v_sl) + c);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");

    const int r = lane / P;           // this lane's query
    const int part = lane % P;        // which 64 / P dimensions of the row it holds
    const uint32_t group_mask = (P == 1 ? 1u : ((1u << P) - 1u)) << (lane & ~(P - 1));
    const bool active = r < lq;
    const int rg = r + off;           // its position in the sample
    const bool self_row = active && a.padded_query_self && rg >= valid_len && rg < ns_start;
    uint4 qraw[CPL];
    if (active && !self_row) {
#pragma unroll
        for (int c = 0; c < CPL; ++c)
            qraw[c] = reinterpret_cast<const uint4*>(qp + static_cast<int64_t>(r) * a.q_sl)[part * CPL + c];
    }
    // every lane waits for its own copies, then the warp agrees that K and V are in shared memory
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncwarp();
    if (!active) return;
    if (self_row) {   // padded query: its own value row
        const uint4* src = reinterpret_cast<const uint4*>(vp + static_cast<int64_t>(rg) * a.v_sl);
        uint4* dst = reinterpret_cast<uint4*>(op + static_cast<int64_t>(r) * a.o_sl);
#pragma unroll
        for (int c = 0; c < CPL; ++c) dst[part * CPL + c] = src[part * CPL + c];
        return;
    }

    float2 q[CPL * 4];
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
        float2 f[4];
        Vec16<T>::unpack2(qraw[c], f);
#pragma unroll
        for (int e = 0; e < 4; ++e) q[4 * c + e] = __fmul2_rn(f[e], make_float2(a.scale_log2, a.scale_log2));
    }
    float2 acc[CPL * 4];
#pragma unroll
    for (int i = 0; i < CPL * 4; ++i) acc[i] = make_float2(0.f, 0.f);
    float m = -INFINITY, l = 0.f;
    const int k_end = causal ? min(lk, rg + 1) : lk;
    for (int j = 0; j < k_end; ++j) {
        if (!attn_visible(rg, j, valid_len, ns_start, lk, causal)) continue;   // same decision in the whole group
        float2 dot = make_float2(0.f, 0.f);
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
            float2 f[4];
            Vec16<T>::unpack2(ks[j * kChunks + part * CPL + c], f);
#pragma unroll
            for (int e = 0; e < 4; ++e) dot = __ffma2_rn(q[4 * c + e], f[e], dot);
        }
        float s = dot.x + dot.y;
#pragma unroll
        for (int o = 1; o < P; o <<= 1) s += __shfl_xor_sync(group_mask, s, o);
        const float m_new = fmaxf(m, s);
        const float corr = ex2(m - m_new);      // first key: exp2(-inf) = 0
        const float p = ex2(s - m_new);
        l = l * corr + p;
        m = m_new;
        const float2 corr2 = make_float2(corr, corr);
        const float2 p2 = make_float2(p, p);
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
            float2 f[4];
            Vec16<T>::unpack2(vs[j * kChunks + part * CPL + c], f);
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[4 * c + e] = __ffma2_rn(f[e], p2, __fmul2_rn(acc[4 * c + e], corr2));
        }
    }
    const float inv1 = l > 0.f ? 1.0f / l : 0.f;
    const float2 inv = make_float2(inv1, inv1);
    uint4* dst = reinterpret_cast<uint4*>(op + static_cast<int64_t>(r) * a.o_sl);
#pragma unroll
    for (int c = 0; c < CPL; ++c) {
        float2 f[4];
#pragma unroll
        for (int e = 0; e < 4; ++e) f[e] = __fmul2_rn(acc[4 * c + e], inv);
        dst[part * CPL + c] = Vec16<T>::pack2(f);
    }
}

template <typename T>
void launch_small(const AttnArgs& a, int64_t grid, cudaStream_t stream) {
    // upper bound of the query rows a warp serves (the keys always fit: kMaxL rows of shared memory per warp)
    const int longest = a.cu_rows_q != nullptr ? a.Lq : (a.Lq > a.Lk ? a.Lq : a.Lk);
    const unsigned g = static_cast<unsigned>(grid);
    if (longest <= kMaxL / 4) attn_small_kernel<T, 4><<<g, kWarps * 32, 0, stream>>>(a);
    else if (longest <= kMaxL / 2) attn_small_kernel<T, 2><<<g, kWarps * 32, 0, stream>>>(a);
    else attn_small_kernel<T, 1><<<g, kWarps * 32, 0, stream>>>(a);
}

}  // namespace

bool attn_small_supported(const AttnArgs& a, int head_dim, int max_lq, int max_lk) {
    return head_dim == kD && a.key_valid == nullptr && max_lq <= kMaxL && max_lk <= kMaxL;
}

int attn_small_forward(const AttnArgs& a, int dtype, cudaStream_t stream) {
    const int64_t pairs = static_cast<int64_t>(a.B) * a.H;
    const int64_t grid = (pairs + kWarps - 1) / kWarps;
    if (grid > 0x7FFFFFFFll) return TB200_ERR_SHAPE;
    if (dtype == TB200_BF16) launch_small<__nv_bfloat16>(a, grid, stream);
    else launch_small<__half>(a, grid, stream);
    count_launch();
    return launch_status();
}

}  // namespace tb200
