// Varlen masked attention forward, broad-coverage kernel (head_dim 32 / 64 / 128, bf16 / fp16,
// any strides, padded or packed batches).  Online softmax in registers, fp32 accumulation,
// warp-level mma.sync m16n8k16 tiles fed by cp.async double buffering.  KV tiles that hold no
// visible key for the query tile are skipped, and query tiles that lie wholly inside the padded
// region only copy their value rows.  The tcgen05 kernel covers the head_dim-64 bf16 hot shape;
// this one covers everything else.
#include "attn_common.cuh"
#include "tb200_common.cuh"

namespace tb200 {
void count_launch();

namespace {

constexpr int kBM = 64;  // query rows per CTA (16 per warp)
constexpr int kBN = 64;
constexpr int kKvStages = 2;  // K / V ring depth (three stages were measured: no faster)
constexpr int kThreads = 128;

template <int D>
__device__ __forceinline__ int swz(int row, int chunk) {  // element offset of a 16-byte chunk
    constexpr int CH = D / 8;
    if (CH >= 8) return row * D + ((chunk ^ (row & 7)) << 3);
    if (CH == 4) return row * D + ((chunk ^ ((row >> 1) & 3)) << 3);
    return row * D + ((chunk ^ ((row >> 2) & 1)) << 3);
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(smem));
    const int bytes = pred ? 16 : 0;  // src-size 0 -> zero fill
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(s), "l"(gmem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t (&r)[4], const void* p) {
    const uint32_t s = static_cast<uint32_t>(__cvta_generic_to_shared(p));
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0, %1, %2, %3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3])
                 : "r"(s));
}

template <typename T>
__device__ __forceinline__ void mma16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <>
__device__ __forceinline__ void mma16816<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0,
                                                        uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <>
__device__ __forceinline__ void mma16816<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <typename T>
__device__ __forceinline__ uint32_t pack2(float lo, float hi);
template <>
__device__ __forceinline__ uint32_t pack2<__nv_bfloat16>(float lo, float hi) {
    __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}
template <>
__device__ __forceinline__ uint32_t pack2<__half>(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&h);
}

// rows [row0, row0 + 64) of a [*, D] strided matrix -> swizzled shared tile; rows >= n_rows are zero
template <typename T, int D>
__device__ __forceinline__ void load_tile(T* smem, const T* gmem, int64_t stride_l, int row0, int n_rows, int tid) {
    constexpr int CH = D / 8;
    for (int i = tid; i < kBN * CH; i += kThreads) {
        const int r = i / CH;
        const int c = i - r * CH;
        const bool ok = row0 + r < n_rows;
        const T* src = gmem + static_cast<int64_t>(ok ? row0 + r : 0) * stride_l + c * 8;
        cp_async16(smem + swz<D>(r, c), src, ok);
    }
}

template <typename T, int D>
__global__ void __launch_bounds__(kThreads, D <= 64 ? 4 : 2) attn_mma_kernel(const AttnArgs a) {
    extern __shared__ __align__(128) uint8_t smem_raw[];
    T* sQ = reinterpret_cast<T*>(smem_raw);
    T* sK = sQ + kBM * D;              // kKvStages stages
    T* sV = sK + kKvStages * kBN * D;  // kKvStages stages

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    const int g = lane >> 2;
    const int t = lane & 3;
    const int b = blockIdx.z;
    const int h = blockIdx.y;
    const int m0 = blockIdx.x * kBM;

    int lq = a.Lq, lk = a.Lk;
    int64_t row_base = 0;      // first key / value row of the sample (packed)
    int64_t q_base = 0;        // first query / output row of the sample (packed)
    int off = 0;               // causal alignment: query r sees keys <= r + off
    if (a.cu_rows != nullptr) {
        row_base = a.cu_rows[b];
        lq = lk = a.cu_rows[b + 1] - static_cast<int32_t>(row_base);
        q_base = row_base;
        if (a.cu_rows_q != nullptr) {   // the queries are the last lq rows of the sample
            q_base = a.cu_rows_q[b];
            lq = a.cu_rows_q[b + 1] - static_cast<int32_t>(q_base);
            off = max(lk - lq, 0);
        }
    }
    if (m0 >= lq) return;
    const bool packed = a.cu_rows != nullptr;
    const T* q = static_cast<const T*>(a.q) + (packed ? q_base * a.q_sl : b * a.q_sb) + h * a.q_sh;
    const T* k = static_cast<const T*>(a.k) + (packed ? row_base * a.k_sl : b * a.k_sb) + h * a.k_sh;
    const T* v = static_cast<const T*>(a.v) + (packed ? row_base * a.v_sl : b * a.v_sb) + h * a.v_sh;
    T* o = static_cast<T*>(a.o) + (packed ? q_base * a.o_sl : b * a.o_sb) + h * a.o_sh;

    const int valid_len = (a.seq_len != nullptr && !packed) ? min(max(a.seq_len[b], 0), lk) : lk;
    const int ns_start = packed ? lk : min(a.ns_start, lk);
    const bool causal = a.causal != 0;
    const bool self_rows = a.padded_query_self != 0;
    const int m_end = min(m0 + kBM, lq);
    // queries in [valid_len, ns_start) are padded; they return their value row
    const uint8_t* kvalid = (a.key_valid != nullptr && !packed) ? a.key_valid + static_cast<int64_t>(b) * lk : nullptr;
    const bool tile_all_padded = kvalid == nullptr && self_rows && m0 >= valid_len && m_end <= ns_start;

    float acc_o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc_o[j][e] = 0.f;
    float row_m[2] = {-INFINITY, -INFINITY};
    float row_l[2] = {0.f, 0.f};

    if (!tile_all_padded) {
        // key tiles that can hold a visible key for this query tile
        const int kv_end = causal ? min(lk, m_end + off) : lk;
        const int n_tiles = (kv_end + kBN - 1) / kBN;
        auto tile_live = [&](int n) {
            const int n0 = n * kBN;
            return kvalid != nullptr || n0 < valid_len || n0 + kBN > ns_start;
        };
        int first = 0;
        while (first < n_tiles && !tile_live(first)) ++first;

        // K / V tiles go through a ring of kKvStages stages: kKvStages - 1 tiles are in flight while one is
        // being used (with a handful of queries per sample the kernel is a stream over K and V)
        auto next_live = [&](int n) {
            ++n;
            while (n < n_tiles && !tile_live(n)) ++n;
            return n;
        };
        load_tile<T, D>(sQ, q, a.q_sl, m0, lq, tid);
        int to_load = first;               // next tile to request
        int load_stage = 0;
#pragma unroll
        for (int i = 0; i < kKvStages - 1; ++i) {
            if (to_load < n_tiles) {
                load_tile<T, D>(sK + load_stage * kBN * D, k, a.k_sl, to_load * kBN, lk, tid);
                load_tile<T, D>(sV + load_stage * kBN * D, v, a.v_sl, to_load * kBN, lk, tid);
                to_load = next_live(to_load);
                load_stage = load_stage + 1 == kKvStages ? 0 : load_stage + 1;
            }
            cp_async_commit();
        }

        uint32_t qf[D / 16][4];
        bool q_loaded = false;
        const bool warp_has_rows = m0 + warp * 16 < lq;
        int stage = 0;
        for (int n = first; n < n_tiles;) {
            const int next = next_live(n);
            if (to_load < n_tiles) {       // refill the stage that was released at the end of the last iteration
                load_tile<T, D>(sK + load_stage * kBN * D, k, a.k_sl, to_load * kBN, lk, tid);
                load_tile<T, D>(sV + load_stage * kBN * D, v, a.v_sl, to_load * kBN, lk, tid);
                to_load = next_live(to_load);
                load_stage = load_stage + 1 == kKvStages ? 0 : load_stage + 1;
            }
            cp_async_commit();
            cp_async_wait<kKvStages - 1>();
            __syncthreads();

            // a warp whose 16 query rows all lie past the sample's last query (few queries against many keys) only
            // helps with the loads and the barriers
            if (warp_has_rows) {
            if (!q_loaded) {
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)
                    ldsm_x4(qf[kk], sQ + swz<D>(warp * 16 + (lane & 15), kk * 2 + (lane >> 4)));
                q_loaded = true;
            }
            const T* cK = sK + stage * kBN * D;
            const T* cV = sV + stage * kBN * D;

            // S = Q K^T
            float s[kBN / 8][4];
#pragma unroll
            for (int j = 0; j < kBN / 8; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
#pragma unroll
                for (int jp = 0; jp < kBN / 16; ++jp) {
                    uint32_t kb[4];
                    const int mi = lane >> 3;
                    ldsm_x4(kb, cK + swz<D>(jp * 16 + (mi >> 1) * 8 + (lane & 7), kk * 2 + (mi & 1)));
                    mma16816<T>(s[2 * jp], qf[kk], kb[0], kb[1]);
                    mma16816<T>(s[2 * jp + 1], qf[kk], kb[2], kb[3]);
                }
            }

            // mask (only tiles that touch a boundary)
            const int n0 = n * kBN;
            const bool full = (n0 + kBN <= valid_len || n0 >= ns_start) && n0 + kBN <= lk && (!causal || n0 + kBN - 1 <= m0 + off);
            if (kvalid != nullptr) {  // arbitrary key-padding pattern: one byte per key
#pragma unroll
                for (int j = 0; j < kBN / 8; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int r = m0 + warp * 16 + g + ((e >> 1) << 3);
                        const int c = n0 + j * 8 + 2 * t + (e & 1);
                        const bool vis = c < lk && kvalid[c] != 0 && (!causal || c <= r + off);
                        if (!vis) s[j][e] = -INFINITY;
                    }
            } else if (!full) {
#pragma unroll
                for (int j = 0; j < kBN / 8; ++j)
#pragma unroll
                    for (int e = 0; e < 4; ++e) {
                        const int r = m0 + warp * 16 + g + ((e >> 1) << 3);
                        const int c = n0 + j * 8 + 2 * t + (e & 1);
                        if (!attn_visible(r + off, c, valid_len, ns_start, lk, causal)) s[j][e] = -INFINITY;
                    }
            }

            // online softmax (rows g and g + 8 of this warp's 16)
#pragma unroll
            for (int hr = 0; hr < 2; ++hr) {
                float mx = row_m[hr];
#pragma unroll
                for (int j = 0; j < kBN / 8; ++j) mx = fmaxf(mx, fmaxf(s[j][2 * hr], s[j][2 * hr + 1]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_use = mx == -INFINITY ? 0.f : mx;
                const float corr = exp2f((row_m[hr] - m_use) * a.scale_log2);  // exp2(-inf) = 0 on the first tile
                row_m[hr] = mx;
                float sum = 0.f;
                const float ms = m_use * a.scale_log2;
#pragma unroll
                for (int j = 0; j < kBN / 8; ++j) {
                    const float p0 = exp2f(fmaf(s[j][2 * hr], a.scale_log2, -ms));
                    const float p1 = exp2f(fmaf(s[j][2 * hr + 1], a.scale_log2, -ms));
                    s[j][2 * hr] = p0;
                    s[j][2 * hr + 1] = p1;
                    sum += p0 + p1;
                }
                row_l[hr] = row_l[hr] * corr + sum;
#pragma unroll
                for (int j = 0; j < D / 8; ++j) {
                    acc_o[j][2 * hr] *= corr;
                    acc_o[j][2 * hr + 1] *= corr;
                }
            }

            // O += P V
#pragma unroll
            for (int kk = 0; kk < kBN / 16; ++kk) {
                uint32_t pa[4];
                pa[0] = pack2<T>(s[2 * kk][0], s[2 * kk][1]);
                pa[1] = pack2<T>(s[2 * kk][2], s[2 * kk][3]);
                pa[2] = pack2<T>(s[2 * kk + 1][0], s[2 * kk + 1][1]);
                pa[3] = pack2<T>(s[2 * kk + 1][2], s[2 * kk + 1][3]);
#pragma unroll
                for (int jp = 0; jp < D / 16; ++jp) {
                    uint32_t vb[4];
                    const int mi = lane >> 3;
                    ldsm_x4_t(vb, cV + swz<D>(kk * 16 + (mi & 1) * 8 + (lane & 7), jp * 2 + (mi >> 1)));
                    mma16816<T>(acc_o[2 * jp], pa, vb[0], vb[1]);
                    mma16816<T>(acc_o[2 * jp + 1], pa, vb[2], vb[3]);
                }
            }
            }  // warp_has_rows
            __syncthreads();  // everyone is done with this stage before it is refilled
            stage = stage + 1 == kKvStages ? 0 : stage + 1;
            n = next;
        }
        cp_async_wait<0>();

        // normalise; rows without a visible key stay zero
#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            float l = row_l[hr];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            const float inv = l > 0.f ? 1.0f / l : 0.f;
#pragma unroll
            for (int j = 0; j < D / 8; ++j) {
                acc_o[j][2 * hr] *= inv;
                acc_o[j][2 * hr + 1] *= inv;
            }
        }
        __syncthreads();
        // stage the output tile in the Q buffer for 16-byte stores
#pragma unroll
        for (int j = 0; j < D / 8; ++j) {
            const int r0 = warp * 16 + g;
            *reinterpret_cast<uint32_t*>(sQ + swz<D>(r0, j) + 2 * t) = pack2<T>(acc_o[j][0], acc_o[j][1]);
            *reinterpret_cast<uint32_t*>(sQ + swz<D>(r0 + 8, j) + 2 * t) = pack2<T>(acc_o[j][2], acc_o[j][3]);
        }
        __syncthreads();
    }

    constexpr int CH = D / 8;
    for (int i = tid; i < kBM * CH; i += kThreads) {
        const int r = i / CH;
        const int c = i - r * CH;
        const int row = m0 + r;
        if (row >= lq) continue;
        uint4 val;
        const bool padded_q = kvalid != nullptr ? kvalid[row] == 0 : (row >= valid_len && row < ns_start);
        if (self_rows && padded_q) {
            val = *reinterpret_cast<const uint4*>(v + static_cast<int64_t>(row) * a.v_sl + c * 8);
        } else {
            val = *reinterpret_cast<const uint4*>(sQ + swz<D>(r, c));
        }
        *reinterpret_cast<uint4*>(o + static_cast<int64_t>(row) * a.o_sl + c * 8) = val;
    }
}

// ------------------------------------------------------------------------------------------------
// Samples of at most 16 rows (head_dim 64): one warp per (sample, head), the whole problem is one
// 16 x 16 score tile: 8 MMAs for Q K^T, a register softmax, 8 MMAs for P V.  Same masks and layouts as the
// kernel above; Lq == Lk <= 16 (packed samples or padded batches).
// ------------------------------------------------------------------------------------------------
constexpr int kTinyL = 16;
constexpr int kTinyWarps = 4;

template <typename T>
__global__ void __launch_bounds__(kTinyWarps * 32)
attn_tiny_kernel(const AttnArgs a) {
    constexpr int D = 64;
    constexpr int CH = D / 8;
    __shared__ __align__(128) T tiles[kTinyWarps][3][kTinyL * D];   // Q (later the output), K, V per warp
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;
    const int t = lane & 3;
    const int64_t pair = static_cast<int64_t>(blockIdx.x) * kTinyWarps + warp;
    if (pair >= static_cast<int64_t>(a.B) * a.H) return;
    const int b = static_cast<int>(pair / a.H);
    const int h = static_cast<int>(pair - static_cast<int64_t>(b) * a.H);

    const bool packed = a.cu_rows != nullptr;
    int lq = a.Lq, lk = a.Lk;
    int64_t row_base = 0;
    if (packed) {
        row_base = a.cu_rows[b];
        lq = lk = a.cu_rows[b + 1] - static_cast<int32_t>(row_base);
    }
    lq = min(lq, kTinyL);
    lk = min(lk, kTinyL);
    if (lq <= 0) return;   // empty sample: nothing to read or write (uniform over the warp)
    const int valid_len = (a.seq_len != nullptr && !packed) ? min(max(a.seq_len[b], 0), lk) : lk;
    const int ns_start = packed ? lk : min(a.ns_start, lk);
    const bool causal = a.causal != 0;
    const T* q = static_cast<const T*>(a.q) + (packed ? row_base * a.q_sl : static_cast<int64_t>(b) * a.q_sb) + static_cast<int64_t>(h) * a.q_sh;
    const T* k = static_cast<const T*>(a.k) + (packed ? row_base * a.k_sl : static_cast<int64_t>(b) * a.k_sb) + static_cast<int64_t>(h) * a.k_sh;
    const T* v = static_cast<const T*>(a.v) + (packed ? row_base * a.v_sl : static_cast<int64_t>(b) * a.v_sb) + static_cast<int64_t>(h) * a.v_sh;
    T* o = static_cast<T*>(a.o) + (packed ? row_base * a.o_sl : static_cast<int64_t>(b) * a.o_sb) + static_cast<int64_t>(h) * a.o_sh;

    T* sQ = tiles[warp][0];
    T* sK = tiles[warp][1];
    T* sV = tiles[warp][2];
    // 16 rows x 8 pieces per matrix: four pieces per lane and matrix, rows past the sample are zero-filled
#pragma unroll
    for (int i = lane; i < kTinyL * CH; i += 32) {
        const int r = i / CH;
        const int c = i - r * CH;
        cp_async16(sQ + swz<D>(r, c), q + static_cast<int64_t>(r < lq ? r : 0) * a.q_sl + c * 8, r < lq);
        cp_async16(sK + swz<D>(r, c), k + static_cast<int64_t>(r < lk ? r : 0) * a.k_sl + c * 8, r < lk);
        cp_async16(sV + swz<D>(r, c), v + static_cast<int64_t>(r < lk ? r : 0) * a.v_sl + c * 8, r < lk);
    }
    cp_async_commit();
    cp_async_wait<0>();
    __syncwarp();

    // S = Q K^T: 16 x 16
    float s[2][4];
#pragma unroll
    for (int j = 0; j < 2; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
    const int mi = lane >> 3;
#pragma unroll
    for (int kk = 0; kk < D / 16; ++kk) {
        uint32_t qf[4], kb[4];
        ldsm_x4(qf, sQ + swz<D>(lane & 15, kk * 2 + (lane >> 4)));
        ldsm_x4(kb, sK + swz<D>((mi >> 1) * 8 + (lane & 7), kk * 2 + (mi & 1)));
        mma16816<T>(s[0], qf, kb[0], kb[1]);
        mma16816<T>(s[1], qf, kb[2], kb[3]);
    }
    // mask, softmax of rows g and g + 8 (each row lives in the four lanes of a quad)
    float inv_l[2];
#pragma unroll
    for (int hr = 0; hr < 2; ++hr) {
        const int r = g + 8 * hr;
        float mx = -INFINITY;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const int c = j * 8 + 2 * t + e;
                if (!attn_visible(r, c, valid_len, ns_start, lk, causal)) s[j][2 * hr + e] = -INFINITY;
                mx = fmaxf(mx, s[j][2 * hr + e]);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float ms = (mx == -INFINITY ? 0.f : mx) * a.scale_log2;
        float sum = 0.f;
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const float p = exp2f(s[j][2 * hr + e] * a.scale_log2 - ms);   // exp2(-inf) = 0
                s[j][2 * hr + e] = p;
                sum += p;
            }
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        inv_l[hr] = sum > 0.f ? 1.0f / sum : 0.f;
    }
    // O = P V: the 16 x 16 probabilities are one A fragment
    uint32_t pa[4];
    pa[0] = pack2<T>(s[0][0], s[0][1]);
    pa[1] = pack2<T>(s[0][2], s[0][3]);
    pa[2] = pack2<T>(s[1][0], s[1][1]);
    pa[3] = pack2<T>(s[1][2], s[1][3]);
    float acc[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j)
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
#pragma unroll
    for (int jp = 0; jp < D / 16; ++jp) {
        uint32_t vb[4];
        ldsm_x4_t(vb, sV + swz<D>((mi & 1) * 8 + (lane & 7), jp * 2 + (mi >> 1)));
        mma16816<T>(acc[2 * jp], pa, vb[0], vb[1]);
        mma16816<T>(acc[2 * jp + 1], pa, vb[2], vb[3]);
    }
    __syncwarp();   // every lane has read its Q fragments: the Q tile becomes the output staging tile
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
        *reinterpret_cast<uint32_t*>(sQ + swz<D>(g, j) + 2 * t) = pack2<T>(acc[j][0] * inv_l[0], acc[j][1] * inv_l[0]);
        *reinterpret_cast<uint32_t*>(sQ + swz<D>(g + 8, j) + 2 * t) = pack2<T>(acc[j][2] * inv_l[1], acc[j][3] * inv_l[1]);
    }
    __syncwarp();
    const bool self_rows = a.padded_query_self != 0;
#pragma unroll
    for (int i = lane; i < kTinyL * CH; i += 32) {
        const int r = i / CH;
        const int c = i - r * CH;
        if (r >= lq) continue;
        const bool padded_q = self_rows && r >= valid_len && r < ns_start;
        const uint4 val = padded_q ? *reinterpret_cast<const uint4*>(v + static_cast<int64_t>(r) * a.v_sl + c * 8)
                                   : *reinterpret_cast<const uint4*>(sQ + swz<D>(r, c));
        *reinterpret_cast<uint4*>(o + static_cast<int64_t>(r) * a.o_sl + c * 8) = val;
    }
}

// ------------------------------------------------------------------------------------------------
// Packed samples with FEW queries against many keys (head_dim 64): after the pyramid has chosen the rows it
// keeps, a sample's queries are its last handful of rows, while its keys are all of them.  A 64-row query tile
// is then almost empty and the launch is a stream over K and V.  Here one warp owns a (sample, head): its 16
// query rows live in registers as MMA fragments, the keys and values pass through a private ring of 16-row
// tiles filled by cp.async (no block-wide barrier anywhere), and every tile is 8 MMAs for Q K^T, an online
// softmax in registers and 8 MMAs for P V.  Samples with more than 16 queries take their query tiles one after
// the other in the same warp.  Masks: packed batches only (every key valid), causal aligned at the end when
// the queries have their own offsets.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ float fq_ex2(float x) {   // 2^x, -inf -> 0
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

constexpr int kFqWarps = 4;
constexpr int kFqStages = 3;
constexpr int kFqRows = 16;    // keys per tile = queries per tile

template <typename T>
__global__ void __launch_bounds__(kFqWarps * 32, 4)
attn_fewq_kernel(const AttnArgs a) {
    constexpr int D = 64;
    constexpr int CH = D / 8;
    extern __shared__ __align__(128) uint8_t fq_smem[];
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int g = lane >> 2;
    const int t = lane & 3;
    const int mi = lane >> 3;
    const int64_t pair = static_cast<int64_t>(blockIdx.x) * kFqWarps + warp;
    if (pair >= static_cast<int64_t>(a.B) * a.H) return;
    const int b = static_cast<int>(pair / a.H);
    const int h_own = static_cast<int>(pair - static_cast<int64_t>(b) * a.H);

    const int64_t row_base = a.cu_rows[b];
    const int lk = a.cu_rows[b + 1] - static_cast<int32_t>(row_base);
    int64_t q_base = row_base;
    int lq = lk;
    if (a.cu_rows_q != nullptr) {
        q_base = a.cu_rows_q[b];
        lq = a.cu_rows_q[b + 1] - static_cast<int32_t>(q_base);
    }
    if (lq <= 0 || lk <= 0) return;   // uniform over the warp
    const int off = max(lk - lq, 0);
    const bool causal = a.causal != 0;
    // this warp's ring: kFqStages x (K tile, V tile) of 16 rows x 64
    T* ring = reinterpret_cast<T*>(fq_smem) + static_cast<size_t>(warp) * kFqStages * 2 * kFqRows * D;

    // Work split.  A sample of at most 16 queries: warp w owns head w of the block's heads and its only query tile.
    // A sample with more: when the block's warps all belong to one sample (H a multiple of the warps per
    // block), its (head, query tile) pairs are dealt to the warps head by head, warp w taking pairs w, w + 4, ...;
    // warps that work on the same head then read the same keys and values at about the same time, so all but
    // one of them are served by the L2 instead of re-reading a long sample from HBM once per query tile, and no
    // warp idles when a head has fewer query tiles than the block has warps.
    const bool together = lq > kFqRows && a.H % kFqWarps == 0;
    const int h_first = together ? h_own - warp : h_own;
    const int n_qt = (lq + kFqRows - 1) / kFqRows;
    const int n_items = together ? kFqWarps * n_qt : n_qt;

    for (int item = together ? warp : 0; item < n_items; item += together ? kFqWarps : 1) {
    const int h = h_first + (together ? item / n_qt : 0);
    const int r0 = (together ? item % n_qt : item) * kFqRows;
    const T* q = static_cast<const T*>(a.q) + q_base * a.q_sl + static_cast<int64_t>(h) * a.q_sh;
    const T* k = static_cast<const T*>(a.k) + row_base * a.k_sl + static_cast<int64_t>(h) * a.k_sh;
    const T* v = static_cast<const T*>(a.v) + row_base * a.v_sl + static_cast<int64_t>(h) * a.v_sh;
    T* o = static_cast<T*>(a.o) + q_base * a.o_sl + static_cast<int64_t>(h) * a.o_sh;
    auto issue = [&](int tile) {   // rows [16 tile, 16 tile + 16) of K and V; rows past the sample are zero
        T* sK = ring + static_cast<size_t>(tile % kFqStages) * 2 * kFqRows * D;
        T* sV = sK + kFqRows * D;
#pragma unroll
        for (int i = lane; i < kFqRows * CH; i += 32) {
            const int r = i / CH;
            const int c = i - r * CH;
            const int row = tile * kFqRows + r;
            const bool ok = row < lk;
            cp_async16(sK + swz<D>(r, c), k + static_cast<int64_t>(ok ? row : 0) * a.k_sl + c * 8, ok);
            cp_async16(sV + swz<D>(r, c), v + static_cast<int64_t>(ok ? row : 0) * a.v_sl + c * 8, ok);
        }
    };

    {
        // keys the tile's last existing query can see
        const int q_last = min(r0 + kFqRows, lq) - 1;
        const int kv_end = causal ? min(lk, q_last + off + 1) : lk;
        const int n_tiles = (kv_end + kFqRows - 1) / kFqRows;
#pragma unroll
        for (int s0 = 0; s0 < kFqStages - 1; ++s0) {
            if (s0 < n_tiles) issue(s0);
            cp_async_commit();
        }
        // Q fragments straight from global memory: rows r0 + g and r0 + g + 8, columns 16 kk + 2 t (+ 8)
        uint32_t qf[D / 16][4];
        {
            const bool ok0 = r0 + g < lq, ok1 = r0 + g + 8 < lq;
            const T* q0 = q + static_cast<int64_t>(ok0 ? r0 + g : 0) * a.q_sl + 2 * t;
            const T* q1 = q + static_cast<int64_t>(ok1 ? r0 + g + 8 : 0) * a.q_sl + 2 * t;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                qf[kk][0] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + kk * 16) : 0u;
                qf[kk][1] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + kk * 16) : 0u;
                qf[kk][2] = ok0 ? *reinterpret_cast<const uint32_t*>(q0 + kk * 16 + 8) : 0u;
                qf[kk][3] = ok1 ? *reinterpret_cast<const uint32_t*>(q1 + kk * 16 + 8) : 0u;
            }
        }
        float acc[D / 8][4];
#pragma unroll
        for (int j = 0; j < D / 8; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[j][e] = 0.f;
        float m_run[2] = {-INFINITY, -INFINITY};   // running maxima of rows g, g + 8 (raw scores)
        float l_run[2] = {0.f, 0.f};               // this lane's share of the running sums

        for (int jt = 0; jt < n_tiles; ++jt) {
            if (jt + kFqStages - 1 < n_tiles) issue(jt + kFqStages - 1);
            cp_async_commit();
            cp_async_wait<kFqStages - 1>();
            __syncwarp();
            const T* sK = ring + static_cast<size_t>(jt % kFqStages) * 2 * kFqRows * D;
            const T* sV = sK + kFqRows * D;
            float s[2][4];
#pragma unroll
            for (int j = 0; j < 2; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) s[j][e] = 0.f;
#pragma unroll
            for (int kk = 0; kk < D / 16; ++kk) {
                uint32_t kb[4];
                ldsm_x4(kb, sK + swz<D>((mi >> 1) * 8 + (lane & 7), kk * 2 + (mi & 1)));
                mma16816<T>(s[0], qf[kk], kb[0], kb[1]);
                mma16816<T>(s[1], qf[kk], kb[2], kb[3]);
            }
            const int c0 = jt * kFqRows;
            // only the tiles on the causal edge and the sample's last tile hold keys a query must not see
            const bool edge = (causal && c0 + kFqRows - 1 > r0 + off) || c0 + kFqRows > lk;
            float p_scale[2];
#pragma unroll
            for (int hr = 0; hr < 2; ++hr) {
                const int rg = r0 + g + 8 * hr + off;   // the query's position among the keys
                float mx = -INFINITY;
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const int c = c0 + j * 8 + 2 * t + e;
                        if (edge && (c >= lk || (causal && c > rg))) s[j][2 * hr + e] = -INFINITY;
                        mx = fmaxf(mx, s[j][2 * hr + e]);
                    }
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_run[hr], mx);
                const float ms = (m_new == -INFINITY ? 0.f : m_new) * a.scale_log2;
                const float corr = fq_ex2(m_run[hr] * a.scale_log2 - ms);   // first tile: exp2(-inf) = 0
                m_run[hr] = m_new;
                float sum = 0.f;
#pragma unroll
                for (int j = 0; j < 2; ++j)
#pragma unroll
                    for (int e = 0; e < 2; ++e) {
                        const float p = fq_ex2(s[j][2 * hr + e] * a.scale_log2 - ms);
                        s[j][2 * hr + e] = p;
                        sum += p;
                    }
                l_run[hr] = l_run[hr] * corr + sum;
                p_scale[hr] = corr;
            }
            if (__any_sync(0xffffffffu, p_scale[0] != 1.f || p_scale[1] != 1.f)) {
#pragma unroll
                for (int j = 0; j < D / 8; ++j) {
                    acc[j][0] *= p_scale[0];
                    acc[j][1] *= p_scale[0];
                    acc[j][2] *= p_scale[1];
                    acc[j][3] *= p_scale[1];
                }
            }
            uint32_t pa[4];
            pa[0] = pack2<T>(s[0][0], s[0][1]);
            pa[1] = pack2<T>(s[0][2], s[0][3]);
            pa[2] = pack2<T>(s[1][0], s[1][1]);
            pa[3] = pack2<T>(s[1][2], s[1][3]);
#pragma unroll
            for (int jp = 0; jp < D / 16; ++jp) {
                uint32_t vb[4];
                ldsm_x4_t(vb, sV + swz<D>((mi & 1) * 8 + (lane & 7), jp * 2 + (mi >> 1)));
                mma16816<T>(acc[2 * jp], pa, vb[0], vb[1]);
                mma16816<T>(acc[2 * jp + 1], pa, vb[2], vb[3]);
            }
            __syncwarp();   // the stage is free for the copy issued at the top of the next iteration
        }
        cp_async_wait<0>();   // nothing of this query tile is in flight when the next one restarts the ring
        __syncwarp();

#pragma unroll
        for (int hr = 0; hr < 2; ++hr) {
            float l = l_run[hr];
            l += __shfl_xor_sync(0xffffffffu, l, 1);
            l += __shfl_xor_sync(0xffffffffu, l, 2);
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            const int r = r0 + g + 8 * hr;
            if (r < lq) {
                T* orow = o + static_cast<int64_t>(r) * a.o_sl + 2 * t;
#pragma unroll
                for (int j = 0; j < D / 8; ++j)
                    *reinterpret_cast<uint32_t*>(orow + j * 8) = pack2<T>(acc[j][2 * hr] * inv, acc[j][2 * hr + 1] * inv);
            }
        }
    }
    }   // (head, query tile) pairs
}

template <typename T, int D>
int launch(const AttnArgs& a, int max_lq, cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(kBM + 2 * kKvStages * kBN) * D * sizeof(T);
    const DeviceInfo& dev = device_info();
    static bool attr_set[64] = {};
    if (!attr_set[dev.index]) {
        cudaFuncSetAttribute(attn_mma_kernel<T, D>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        // the kernel is often a stream over K and V (a few queries per sample): room for as many CTAs as fit
        cudaFuncSetAttribute(attn_mma_kernel<T, D>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        attr_set[dev.index] = true;
    }
    dim3 grid((max_lq + kBM - 1) / kBM, a.H, a.B);
    attn_mma_kernel<T, D><<<grid, kThreads, smem, stream>>>(a);
    count_launch();
    return launch_status();
}

}  // namespace

// Samples of at most 16 rows, head_dim 64, no key_valid map: one warp per (sample, head).
bool attn_tiny_supported(const AttnArgs& a, int head_dim, int max_lq, int max_lk) {
    return head_dim == 64 && a.key_valid == nullptr && a.cu_rows_q == nullptr && max_lq <= kTinyL && max_lk <= kTinyL;
}
int attn_tiny_forward(const AttnArgs& a, int dtype, cudaStream_t stream) {
    const int64_t pairs = static_cast<int64_t>(a.B) * a.H;
    const int64_t grid = (pairs + kTinyWarps - 1) / kTinyWarps;
    if (grid > 0x7FFFFFFFll) return TB200_ERR_SHAPE;
    if (dtype == TB200_BF16) attn_tiny_kernel<__nv_bfloat16><<<static_cast<unsigned>(grid), kTinyWarps * 32, 0, stream>>>(a);
    else attn_tiny_kernel<__half><<<static_cast<unsigned>(grid), kTinyWarps * 32, 0, stream>>>(a);
    count_launch();
    return launch_status();
}

// Packed samples with few queries each (head_dim 64, no key_valid map, 4-byte aligned rows): one warp per
// (sample, head) streams the keys and values.
bool attn_fewq_supported(const AttnArgs& a, int head_dim) {
    auto even = [](int64_t x) { return (x & 1) == 0; };
    return head_dim == 64 && a.cu_rows != nullptr && a.key_valid == nullptr && a.padded_query_self == 0 &&
           even(a.q_sl) && even(a.q_sh) && even(a.o_sl) && even(a.o_sh) &&
           (reinterpret_cast<uintptr_t>(a.q) & 3) == 0 && (reinterpret_cast<uintptr_t>(a.o) & 3) == 0;
}
int attn_fewq_forward(const AttnArgs& a, int dtype, cudaStream_t stream) {
    const int64_t pairs = static_cast<int64_t>(a.B) * a.H;
    const int64_t grid = (pairs + kFqWarps - 1) / kFqWarps;
    if (grid > 0x7FFFFFFFll) return TB200_ERR_SHAPE;
    if (grid == 0) return TB200_OK;
    const size_t smem = static_cast<size_t>(kFqWarps) * kFqStages * 2 * kFqRows * 64 * 2;
    const DeviceInfo& dev = device_info();
    static bool attr_set[64] = {};
    if (!attr_set[dev.index]) {
        cudaFuncSetAttribute(attn_fewq_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        cudaFuncSetAttribute(attn_fewq_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        cudaFuncSetAttribute(attn_fewq_kernel<__nv_bfloat16>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        cudaFuncSetAttribute(attn_fewq_kernel<__half>, cudaFuncAttributePreferredSharedMemoryCarveout, 100);
        attr_set[dev.index] = true;
    }
    if (dtype == TB200_BF16) attn_fewq_kernel<__nv_bfloat16><<<static_cast<unsigned>(grid), kFqWarps * 32, smem, stream>>>(a);
    else attn_fewq_kernel<__half><<<static_cast<unsigned>(grid), kFqWarps * 32, smem, stream>>>(a);
    count_launch();
    return launch_status();
}

// Entry used by the C ABI dispatcher in attn_api.cu.  max_lq bounds the query rows of any sample.
int attn_mma_forward(const AttnArgs& a, int head_dim, int dtype, int max_lq, cudaStream_t stream) {
    if (dtype == TB200_BF16) {
        if (head_dim == 32) return launch<__nv_bfloat16, 32>(a, max_lq, stream);
        if (head_dim == 64) return launch<__nv_bfloat16, 64>(a, max_lq, stream);
        if (head_dim == 128) return launch<__nv_bfloat16, 128>(a, max_lq, stream);
    } else if (dtype == TB200_F16) {
        if (head_dim == 32) return launch<__half, 32>(a, max_lq, stream);
        if (head_dim == 64) return launch<__half, 64>(a, max_lq, stream);
        if (head_dim == 128) return launch<__half, 128>(a, max_lq, stream);
    }
    return TB200_ERR_UNSUPPORTED;
}

}  // namespace tb200
