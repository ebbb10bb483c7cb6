// Fused RMSNorm / LayerNorm forward for sm_100a.
//
// HBM-bound: every element is read once and written once.  The main kernel is a
// persistent CTA that streams tiles of whole rows through shared memory with TMA bulk
// copies (the rows of a contiguous [rows, cols] matrix make one contiguous byte range,
// so no tensor map is needed), normalises each row in registers with a sub-warp
// shuffle reduction, overwrites the tile in place and hands it back to TMA for the
// store.  A 4-stage mbarrier ring keeps 3 loads per CTA in flight.
//
// Rows that cannot be moved in 16-byte units fall back to a warp-per-row kernel with
// scalar accesses; it covers every (cols, alignment) combination.
#include "tb200_common.cuh"
#include "tb200_ptx.cuh"

namespace tb200 {
void count_launch();

namespace {

constexpr int kMaxThreads = 256;
constexpr int kWarps = kMaxThreads / 32;
constexpr int kStages = 4;

// Every warp owns a contiguous span of rows and a private 4-stage ring of small tiles
// (a few rows, about 2 KB) with its own mbarriers: lane 0 issues the bulk loads and stores,
// the warp normalises RU rows per lane group at a time (independent shuffle chains), and no
// CTA-wide barrier is ever taken after start-up.  gamma / beta sit in shared memory.
//
// PRE selects an operation fused in front of the statistics:
//   kPreNone  y = norm(x)
//   kPreBias  y = rmsnorm(x + bias)            (RMS only; the bias vector arrives through `beta`)
//   kPreSilu  y = layernorm(silu(x)), the SiLU result rounded to T like the tensor a separate SiLU
//             kernel would have written
enum Pre : int { kPreNone = 0, kPreBias = 1, kPreSilu = 2 };

// SiLU for a value that is rounded to T afterwards: the 16-bit types take the one-MUFU form
// h * tanh(h) + h (h = x / 2, about 11 bits), fp32 the exponential form.
template <typename T>
__device__ __forceinline__ float silu_f(float x) {
    if (sizeof(T) == 4) return x / (1.0f + __expf(-x));
    const float h = 0.5f * x;
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
    return fmaf(h, t, h);
}
__device__ __forceinline__ void prefetch_l1(const void* p) { asm volatile("prefetch.global.L1 [%0];" ::"l"(p)); }
__device__ __forceinline__ uint4 ld_nc_u4(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
template <typename T>
__device__ __forceinline__ float round_to(float v) {
    return to_float<T>(from_float<T>(v));
}
// The same two operations on a pair of values (same bits as the scalar forms, fewer instructions).
template <typename T>
__device__ __forceinline__ float2 silu_pair(float2 x) {
    if (sizeof(T) == 4) return make_float2(silu_f<T>(x.x), silu_f<T>(x.y));
    const float2 h = __fmul2_rn(x, make_float2(0.5f, 0.5f));
    float2 t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t.x) : "f"(h.x));
    asm("tanh.approx.f32 %0, %1;" : "=f"(t.y) : "f"(h.y));
    return __ffma2_rn(h, t, h);
}
template <typename T>
__device__ __forceinline__ float2 round_pair(float2 v) {
    return v;
}
template <>
__device__ __forceinline__ float2 round_pair<__nv_bfloat16>(float2 v) {
    const __nv_bfloat162 h = __float22bfloat162_rn(v);
    const uint32_t w = *reinterpret_cast<const uint32_t*>(&h);
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
template <>
__device__ __forceinline__ float2 round_pair<__half>(float2 v) {
    return __half22float2(__float22half2_rn(v));
}

// Optional stage behind the normalisation (POST): the normalised row, rounded to T, receives one or two
// gathered table rows (each sum rounded to T, like tensor additions), is written to y, and is then
// RMS-normalised with a second weight vector into a second output.  This is the end of the sequence tokenizer
// and the first norm of the first block in one pass over the token matrix:
//   tokens = LayerNorm(SiLU(x)) + time_rows + position_rows;   normed = RMSNorm(tokens)
// With `row_dst` the first output is compacted: row r goes to y[row_dst[r]] when 0 <= row_dst[r] < rows_out and is
// not written at all otherwise, while `normed` still covers every row.
struct PostArgs {
    const void* table_a;
    const int64_t* ids_a;
    int64_t rows_a;
    const void* table_b;   // may be nullptr
    const int64_t* ids_b;
    int64_t rows_b;
    const void* gamma2;
    void* normed;
    float eps2;
    const int32_t* row_dst;   // may be nullptr
    int64_t rows_out;
};

template <typename T, bool LAYER, int CPL, int RU, int PRE, bool POST, bool EXACT>
__global__ void __launch_bounds__(kMaxThreads, 3)
norm_tma_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
                int64_t rows, int cols, float eps, int lanes_per_row, int* __restrict__ status, const PostArgs post) {
    constexpr int N = Vec16<T>::N;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t full_bar[kWarps][kStages];

    const int tid = threadIdx.x;
    const int warp = tid >> 5;
    const int lane = tid & 31;
    // A row wider than one piece per lane always takes the whole warp, and with EXACT its width is then known at
    // compile time as well: every offset below becomes an immediate and the shuffle loops unroll.
    constexpr bool kWholeWarp = CPL > 1;
    const int chunks = (kWholeWarp && EXACT) ? CPL * 32 : cols / N;  // 16-byte chunks per row
    const uint32_t row_bytes = static_cast<uint32_t>(chunks) * 16u;
    const int G = kWholeWarp ? 32 : lanes_per_row;
    const int ng = 32 / G;           // rows handled side by side by one warp instruction
    const int tile_rows = ng * RU;   // rows per tile
    const uint32_t tile_bytes = row_bytes * static_cast<uint32_t>(tile_rows);
    uint8_t* ring = smem + static_cast<size_t>(warp) * kStages * tile_bytes;
    // gamma / beta as fp32: [N / 4][chunks] float4 each, so that a warp's float4 reads are contiguous
    float2* gamma_s = reinterpret_cast<float2*>(smem + static_cast<size_t>(kWarps) * kStages * tile_bytes);
    float2* beta_s = gamma_s + static_cast<size_t>(chunks) * (N / 2);
    float2* gamma2_s = beta_s + static_cast<size_t>(chunks) * (N / 2);   // POST only

    // contiguous, balanced row span of this warp
    const int64_t n_warps = static_cast<int64_t>(gridDim.x) * kWarps;
    const int64_t w = static_cast<int64_t>(blockIdx.x) * kWarps + warp;
    const int64_t row_begin = (w * rows) / n_warps;
    const int64_t row_end = ((w + 1) * rows) / n_warps;
    const int my_rows = static_cast<int>(row_end - row_begin);   // a warp's span is far below 2^31 rows
    const int n_my = (my_rows + tile_rows - 1) / tile_rows;

    auto rows_in = [&](int it) -> int {
        const int left = my_rows - it * tile_rows;
        return left < tile_rows ? left : tile_rows;
    };
    auto issue_load = [&](int it) {
        const int s = it % kStages;
        const uint32_t bytes = static_cast<uint32_t>(rows_in(it)) * row_bytes;
        mbar_expect_tx(&full_bar[warp][s], bytes);
        bulk_load(ring + static_cast<size_t>(s) * tile_bytes,
                  reinterpret_cast<const uint8_t*>(x) + (row_begin + static_cast<int64_t>(it) * tile_rows) * row_bytes, bytes,
                  &full_bar[warp][s]);
    };

    if (lane == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[warp][s], 1);
        fence_mbar_init();
        for (int it = 0; it < n_my && it < kStages; ++it) issue_load(it);
    }
    for (int c = tid; c < chunks; c += kMaxThreads) {
        float2 f[N / 2];
        Vec16<T>::unpack2(reinterpret_cast<const uint4*>(gamma)[c], f);
#pragma unroll
        for (int e = 0; e < N / 2; ++e) gamma_s[((e >> 1) * chunks + c) * 2 + (e & 1)] = f[e];
        if (LAYER || PRE == kPreBias) {
            Vec16<T>::unpack2(reinterpret_cast<const uint4*>(beta)[c], f);
#pragma unroll
            for (int e = 0; e < N / 2; ++e) beta_s[((e >> 1) * chunks + c) * 2 + (e & 1)] = f[e];
        }
        if (POST) {
            Vec16<T>::unpack2(reinterpret_cast<const uint4*>(post.gamma2)[c], f);
#pragma unroll
            for (int e = 0; e < N / 2; ++e) gamma2_s[((e >> 1) * chunks + c) * 2 + (e & 1)] = f[e];
        }
    }
    __syncthreads();

    const int group = lane / G;
    const int lane_g = lane % G;
    const float inv_cols = 1.0f / static_cast<float>(cols);
    const bool compact = POST && post.row_dst != nullptr;

    for (int it = 0; it < n_my; ++it) {
        const int s = it % kStages;
        const uint32_t parity = static_cast<uint32_t>((it / kStages) & 1);
        const int64_t tile_row0 = row_begin + static_cast<int64_t>(it) * tile_rows;
        const int rows_here = rows_in(it);
        uint4* tile = reinterpret_cast<uint4*>(ring + static_cast<size_t>(s) * tile_bytes);
        const bool ok = mbar_wait_sleep(&full_bar[warp][s], parity);
        if (__any_sync(0xffffffffu, !ok)) {  // a load never arrived: report and leave
            if (lane == 0 && status != nullptr) atomicExch(status, 1);
            break;
        }

        // POST: the table rows of this tile are requested into the L1 now, so that the loads behind the
        // normalisation find them there instead of waiting for the L2 one row at a time
        //
        // A lane group whose row lies behind the end of a ragged last tile works on the tile's last row once more:
        // it reads, computes and writes the same values as that row's own group, which keeps every predicate on
        // rows out of the code below.
        int32_t id_a[RU], id_b[RU];   // clamped into tables of fewer than 2^31 rows
        int32_t dst[RU];
        int rr[RU];
#pragma unroll
        for (int u = 0; u < RU; ++u) {
            id_a[u] = id_b[u] = 0;
            dst[u] = -1;
            rr[u] = min(u * ng + group, rows_here - 1);
            if (POST) {
                const int64_t row = tile_row0 + rr[u];
                if (compact) {
                    const int32_t d = post.row_dst[row];
                    dst[u] = (d >= 0 && d < post.rows_out) ? d : -1;
                }
                int64_t ia = post.ids_a[row];
                id_a[u] = static_cast<int32_t>(ia < 0 ? 0 : (ia > post.rows_a - 1 ? post.rows_a - 1 : ia));
                if (post.table_b != nullptr) {
                    int64_t ib = post.ids_b[row];
                    id_b[u] = static_cast<int32_t>(ib < 0 ? 0 : (ib > post.rows_b - 1 ? post.rows_b - 1 : ib));
                }
#pragma unroll
                for (int j = 0; j < CPL; ++j) {
                    const int c = lane_g + j * G;
                    if (EXACT || c < chunks) {
                        prefetch_l1(reinterpret_cast<const uint4*>(post.table_a) + static_cast<int64_t>(id_a[u]) * chunks + c);
                        if (post.table_b != nullptr) prefetch_l1(reinterpret_cast<const uint4*>(post.table_b) + static_cast<int64_t>(id_b[u]) * chunks + c);
                    }
                }
            }
        }

        // packed fp32x2 arithmetic throughout: the kernel is issue-bound, not HBM-bound, otherwise
        float2 v[RU][CPL][N / 2];
        float sum[RU];
        float sq[RU];
#pragma unroll
        for (int u = 0; u < RU; ++u) {
            const uint4* rowp = tile + static_cast<size_t>(rr[u]) * chunks;
            float2 acc = make_float2(0.f, 0.f);
#pragma unroll
            for (int j = 0; j < CPL; ++j) {
                const int c = lane_g + j * G;
                if (EXACT || c < chunks) {
                    Vec16<T>::unpack2(rowp[c], v[u][j]);
                    if (PRE == kPreBias) {
#pragma unroll
                        for (int e = 0; e < N / 2; e += 2) {
                            const float4 b4 = *reinterpret_cast<const float4*>(&beta_s[((e >> 1) * chunks + c) * 2]);
                            v[u][j][e] = __fadd2_rn(v[u][j][e], make_float2(b4.x, b4.y));
                            v[u][j][e + 1] = __fadd2_rn(v[u][j][e + 1], make_float2(b4.z, b4.w));
                        }
                    }
                    if (PRE == kPreSilu) {
#pragma unroll
                        for (int e = 0; e < N / 2; ++e) v[u][j][e] = round_pair<T>(silu_pair<T>(v[u][j][e]));
                    }
                } else {
#pragma unroll
                    for (int e = 0; e < N / 2; ++e) v[u][j][e] = make_float2(0.f, 0.f);
                }
#pragma unroll
                for (int e = 0; e < N / 2; ++e) {
                    if (LAYER) acc = __fadd2_rn(acc, v[u][j][e]);
                    else acc = __ffma2_rn(v[u][j][e], v[u][j][e], acc);
                }
            }
            sum[u] = acc.x + acc.y;
            sq[u] = sum[u];
        }
        if (LAYER) {
            for (int o = G >> 1; o > 0; o >>= 1) {
#pragma unroll
                for (int u = 0; u < RU; ++u) sum[u] += __shfl_xor_sync(0xffffffffu, sum[u], o);
            }
#pragma unroll
            for (int u = 0; u < RU; ++u) {
                const float nm = -sum[u] * inv_cols;
                const float2 nmean = make_float2(nm, nm);
                float2 acc = make_float2(0.f, 0.f);
#pragma unroll
                for (int j = 0; j < CPL; ++j) {
                    const int c = lane_g + j * G;
                    if (EXACT || c < chunks) {
#pragma unroll
                        for (int e = 0; e < N / 2; ++e) {
                            v[u][j][e] = __fadd2_rn(v[u][j][e], nmean);  // keep the centred value
                            acc = __ffma2_rn(v[u][j][e], v[u][j][e], acc);
                        }
                    }
                }
                sq[u] = acc.x + acc.y;
            }
        }
        for (int o = G >> 1; o > 0; o >>= 1) {
#pragma unroll
            for (int u = 0; u < RU; ++u) sq[u] += __shfl_xor_sync(0xffffffffu, sq[u], o);
        }
        __syncwarp();   // every lane has read its rows before any lane overwrites the tile (duplicated rows included)
        float2 inv[RU];
#pragma unroll
        for (int u = 0; u < RU; ++u) {
            const float i1 = rsqrtf(sq[u] * inv_cols + eps);
            inv[u] = make_float2(i1, i1);
        }
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
            const int c = lane_g + j * G;
            if (EXACT || c < chunks) {
                float2 g[N / 2];
                float2 b[N / 2];
#pragma unroll
                for (int e = 0; e < N / 2; e += 2) {
                    const float4 g4 = *reinterpret_cast<const float4*>(&gamma_s[((e >> 1) * chunks + c) * 2]);
                    g[e] = make_float2(g4.x, g4.y);
                    g[e + 1] = make_float2(g4.z, g4.w);
                    if (LAYER) {
                        const float4 b4 = *reinterpret_cast<const float4*>(&beta_s[((e >> 1) * chunks + c) * 2]);
                        b[e] = make_float2(b4.x, b4.y);
                        b[e + 1] = make_float2(b4.z, b4.w);
                    }
                }
#pragma unroll
                for (int u = 0; u < RU; ++u) {
                    {
                        float2 o[N / 2];
#pragma unroll
                        for (int e = 0; e < N / 2; ++e) {
                            if (LAYER) o[e] = __ffma2_rn(__fmul2_rn(v[u][j][e], inv[u]), g[e], b[e]);
                            else o[e] = __fmul2_rn(__fmul2_rn(v[u][j][e], inv[u]), g[e]);
                        }
                        uint4 packed = Vec16<T>::pack2(o);
                        if (POST) {
                            // each sum rounded to T like a tensor addition: the native packed add of the 16-bit types
                            // gives those bits directly (fp32 holds more than twice their precision plus two bits, so
                            // rounding the fp32 sum again changes nothing)
                            packed = Vec16<T>::add_rn(packed, ld_nc_u4(reinterpret_cast<const uint4*>(post.table_a) + static_cast<int64_t>(id_a[u]) * chunks + c));
                            if (post.table_b != nullptr)
                                packed = Vec16<T>::add_rn(packed, ld_nc_u4(reinterpret_cast<const uint4*>(post.table_b) + static_cast<int64_t>(id_b[u]) * chunks + c));
                            Vec16<T>::unpack2(packed, v[u][j]);   // keep the row for the second normalisation
                        }
                        if (!compact) tile[static_cast<size_t>(rr[u]) * chunks + c] = packed;
                        else if (dst[u] >= 0) reinterpret_cast<uint4*>(y)[static_cast<int64_t>(dst[u]) * chunks + c] = packed;
                    }
                }
            }
        }
        if (POST) {
            float sq2[RU];
#pragma unroll
            for (int u = 0; u < RU; ++u) {
                float2 acc = make_float2(0.f, 0.f);
                {
#pragma unroll
                    for (int j = 0; j < CPL; ++j) {
                        if (EXACT || lane_g + j * G < chunks) {
#pragma unroll
                            for (int e = 0; e < N / 2; ++e) acc = __ffma2_rn(v[u][j][e], v[u][j][e], acc);
                        }
                    }
                }
                sq2[u] = acc.x + acc.y;
            }
            for (int o = G >> 1; o > 0; o >>= 1) {
#pragma unroll
                for (int u = 0; u < RU; ++u) sq2[u] += __shfl_xor_sync(0xffffffffu, sq2[u], o);
            }
#pragma unroll
            for (int j = 0; j < CPL; ++j) {
                const int c = lane_g + j * G;
                if (EXACT || c < chunks) {
                    float2 g2[N / 2];
#pragma unroll
                    for (int e = 0; e < N / 2; e += 2) {
                        const float4 g4 = *reinterpret_cast<const float4*>(&gamma2_s[((e >> 1) * chunks + c) * 2]);
                        g2[e] = make_float2(g4.x, g4.y);
                        g2[e + 1] = make_float2(g4.z, g4.w);
                    }
#pragma unroll
                    for (int u = 0; u < RU; ++u) {
                        {
                            const float i2 = rsqrtf(sq2[u] * inv_cols + post.eps2);
                            const float2 inv2 = make_float2(i2, i2);
                            float2 o[N / 2];
#pragma unroll
                            for (int e = 0; e < N / 2; ++e) o[e] = __fmul2_rn(__fmul2_rn(v[u][j][e], inv2), g2[e]);
                            const int64_t row = tile_row0 + rr[u];
                            reinterpret_cast<uint4*>(post.normed)[row * chunks + c] = Vec16<T>::pack2(o);
                        }
                    }
                }
            }
        }

        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            if (!compact) {
                bulk_store(reinterpret_cast<uint8_t*>(y) + tile_row0 * row_bytes, tile,
                           static_cast<uint32_t>(rows_here) * row_bytes);
                bulk_commit();
            }
            // The stage stored one iteration ago is free once its store has read shared memory.
            if (it >= 1 && it - 1 + kStages < n_my) {
                bulk_wait_read<1>();
                issue_load(it - 1 + kStages);
            }
        }
        __syncwarp();
    }
    if (lane == 0) bulk_wait<0>();
}

// Warp per row, scalar accesses, any cols / alignment.
template <typename T, bool LAYER, int PRE>
__global__ void __launch_bounds__(kMaxThreads)
norm_rowwarp_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                    T* __restrict__ y, int64_t rows, int cols, float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * kMaxThreads + threadIdx.x) >> 5;
    const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * kMaxThreads) >> 5;
    const float inv_cols = 1.0f / static_cast<float>(cols);
    auto load = [&](const T* xr, int c) -> float {
        float v = to_float<T>(xr[c]);
        if (PRE == kPreBias) v += to_float<T>(beta[c]);
        if (PRE == kPreSilu) v = round_to<T>(silu_f<T>(v));
        return v;
    };
    for (int64_t r = warp; r < rows; r += n_warps) {
        const T* xr = x + r * cols;
        T* yr = y + r * cols;
        float mean = 0.f;
        if (LAYER) {
            float sum = 0.f;
            for (int c = lane; c < cols; c += 32) sum += load(xr, c);
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            mean = sum * inv_cols;
        }
        float sq = 0.f;
        for (int c = lane; c < cols; c += 32) {
            const float d = load(xr, c) - mean;
            sq = fmaf(d, d, sq);
        }
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        const float inv = rsqrtf(sq * inv_cols + eps);
        for (int c = lane; c < cols; c += 32) {
            const float v = load(xr, c);
            float o;
            if (LAYER) o = fmaf((v - mean) * inv, to_float<T>(gamma[c]), to_float<T>(beta[c]));
            else o = (v * inv) * to_float<T>(gamma[c]);
            yr[c] = from_float<T>(o);
        }
    }
}

// Warp per row for rows wider than the TMA-staged kernel takes (more than 256 16-byte pieces), whole pieces and
// 16-byte aligned bases: a lane walks the pieces lane, lane + 32, ... three times (sum, centred squares, output) and
// keeps them, after the bias / SiLU step, in a shared-memory row of the warp between the passes.  Every lane only
// reads back the pieces it wrote itself, so the passes need no barrier.
template <typename T, bool LAYER, int PRE>
__global__ void __launch_bounds__(kMaxThreads)
norm_rowwarp_vec_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                        T* __restrict__ y, int64_t rows, int cols, float eps) {
    constexpr int N = Vec16<T>::N;
    extern __shared__ __align__(16) uint8_t smem[];
    const int lane = threadIdx.x & 31;
    const int warp_in_cta = threadIdx.x >> 5;
    const int chunks = cols / N;
    uint4* srow = reinterpret_cast<uint4*>(smem) + static_cast<size_t>(warp_in_cta) * chunks;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * kMaxThreads + threadIdx.x) >> 5;
    const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * kMaxThreads) >> 5;
    const float inv_cols = 1.0f / static_cast<float>(cols);
    const uint4* g4 = reinterpret_cast<const uint4*>(gamma);
    const uint4* b4 = reinterpret_cast<const uint4*>(beta);
    for (int64_t row = warp; row < rows; row += n_warps) {
        const uint4* xr = reinterpret_cast<const uint4*>(x + row * cols);
        uint4* yr = reinterpret_cast<uint4*>(y + row * cols);
        float acc = 0.f;   // LayerNorm: sum of the row; RMSNorm: sum of squares
        for (int c = lane; c < chunks; c += 32) {
            uint4 p = ld_nc_u4(xr + c);
            float f[N];
            Vec16<T>::unpack(p, f);
            if (PRE == kPreBias) {
                float b[N];
                Vec16<T>::unpack(b4[c], b);
#pragma unroll
                for (int e = 0; e < N; ++e) f[e] += b[e];
            }
            if (PRE == kPreSilu) {
#pragma unroll
                for (int e = 0; e < N; ++e) f[e] = round_to<T>(silu_f<T>(f[e]));
                p = Vec16<T>::pack(f);
            }
#pragma unroll
            for (int e = 0; e < N; ++e) acc = LAYER ? acc + f[e] : fmaf(f[e], f[e], acc);
            srow[c] = p;   // with a bias: x as it came (x + bias in fp32 does not fit a 16-bit row; the output pass adds it again)
        }
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        float mean = 0.f, sq = acc;
        if (LAYER) {
            mean = acc * inv_cols;
            sq = 0.f;
            for (int c = lane; c < chunks; c += 32) {
                float f[N];
                Vec16<T>::unpack(srow[c], f);
#pragma unroll
                for (int e = 0; e < N; ++e) {
                    const float d = f[e] - mean;
                    sq = fmaf(d, d, sq);
                }
            }
            for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        }
        const float inv = rsqrtf(sq * inv_cols + eps);
        for (int c = lane; c < chunks; c += 32) {
            float f[N], g[N], o[N];
            Vec16<T>::unpack(srow[c], f);
            Vec16<T>::unpack(g4[c], g);
            if (PRE == kPreBias) {
                float b[N];
                Vec16<T>::unpack(b4[c], b);
#pragma unroll
                for (int e = 0; e < N; ++e) f[e] += b[e];
            }
            if (LAYER) {
                float b[N];
                Vec16<T>::unpack(b4[c], b);
#pragma unroll
                for (int e = 0; e < N; ++e) o[e] = fmaf((f[e] - mean) * inv, g[e], b[e]);
            } else {
#pragma unroll
                for (int e = 0; e < N; ++e) o[e] = (f[e] * inv) * g[e];
            }
            yr[c] = Vec16<T>::pack(o);
        }
    }
}

template <typename T, bool LAYER, int CPL, int RU, int PRE, bool POST, bool EXACT>
int launch_tma_exact(const void* x, const void* gamma, const void* beta, void* y, int64_t rows, int cols, float eps,
                     int lanes_per_row, cudaStream_t stream, const PostArgs post) {
    const int N = Vec16<T>::N;
    const int chunks = cols / N;
    const int row_bytes = chunks * 16;
    const int tile_rows = (32 / lanes_per_row) * RU;
    const size_t tile_bytes = static_cast<size_t>(tile_rows) * row_bytes;
    const size_t smem = tile_bytes * kStages * kWarps + static_cast<size_t>(cols) * sizeof(float) * (POST ? 3 : 2);
    const DeviceInfo& dev = device_info();
    static bool attr_set[64] = {};
    if (!attr_set[dev.index]) {
        cudaFuncSetAttribute(norm_tma_kernel<T, LAYER, CPL, RU, PRE, POST, EXACT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             200 * 1024);
        attr_set[dev.index] = true;
    }
    int ctas_per_sm = static_cast<int>((220 * 1024) / (smem + 1024));
    if (ctas_per_sm > 4) ctas_per_sm = 4;
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    int64_t grid = static_cast<int64_t>(dev.sm_count) * ctas_per_sm;
    const int64_t useful = (rows + static_cast<int64_t>(tile_rows) * kWarps - 1) / (static_cast<int64_t>(tile_rows) * kWarps);
    if (grid > useful) grid = useful;
    if (grid < 1) grid = 1;
    norm_tma_kernel<T, LAYER, CPL, RU, PRE, POST, EXACT><<<static_cast<unsigned>(grid), kMaxThreads, smem, stream>>>(
        static_cast<const T*>(x), static_cast<const T*>(gamma), static_cast<const T*>(beta), static_cast<T*>(y), rows,
        cols, eps, lanes_per_row, nullptr, post);
    count_launch();
    return launch_status();
}

// EXACT: the lanes of a row group cover the row's 16-byte pieces exactly, so no lane ever idles.
template <typename T, bool LAYER, int CPL, int RU, int PRE, bool POST = false>
int launch_tma(const void* x, const void* gamma, const void* beta, void* y, int64_t rows, int cols, float eps,
               int lanes_per_row, cudaStream_t stream, const PostArgs post = PostArgs{}) {
    if (cols / Vec16<T>::N == CPL * lanes_per_row)
        return launch_tma_exact<T, LAYER, CPL, RU, PRE, POST, true>(x, gamma, beta, y, rows, cols, eps, lanes_per_row, stream, post);
    return launch_tma_exact<T, LAYER, CPL, RU, PRE, POST, false>(x, gamma, beta, y, rows, cols, eps, lanes_per_row, stream, post);
}

template <typename T, bool LAYER, int PRE>
int norm_dispatch(const void* x, const void* gamma, const void* beta, void* y, int64_t rows, int cols, float eps,
                  cudaStream_t stream) {
    const int N = Vec16<T>::N;
    const bool vec_ok = (cols % N == 0) && aligned16(x) && aligned16(y) && aligned16(gamma) &&
                        ((!LAYER && PRE != kPreBias) || aligned16(beta)) && (cols / N) <= 256;
    if (vec_ok) {
        const int chunks = cols / N;
        int G = 1;
        while (G < 32 && G < chunks) G <<= 1;  // lanes per row: power of two, <= 32
        const int cpl = (chunks + G - 1) / G;
        // RU rows per lane group and tile, so that a lane holds about 4 chunks whatever the row width
        if (cpl <= 1) return launch_tma<T, LAYER, 1, 4, PRE>(x, gamma, beta, y, rows, cols, eps, G, stream);
        if (cpl <= 2) return launch_tma<T, LAYER, 2, 2, PRE>(x, gamma, beta, y, rows, cols, eps, G, stream);
        if (cpl <= 4) return launch_tma<T, LAYER, 4, 1, PRE>(x, gamma, beta, y, rows, cols, eps, G, stream);
        return launch_tma<T, LAYER, 8, 1, PRE>(x, gamma, beta, y, rows, cols, eps, G, stream);
    }
    const DeviceInfo& dev = device_info();
    int64_t blocks = (rows + (kMaxThreads / 32) - 1) / (kMaxThreads / 32);
    const int64_t cap = static_cast<int64_t>(dev.sm_count) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    const bool wide_vec = (cols % N == 0) && aligned16(x) && aligned16(y) && aligned16(gamma) &&
                          ((!LAYER && PRE != kPreBias) || aligned16(beta)) && (cols / N) <= 640;
    if (wide_vec) {   // up to 10 KB of row per warp, 80 KB per block
        const size_t smem = static_cast<size_t>(kMaxThreads / 32) * (cols / N) * 16;
        static bool attr_set[64] = {};
        if (!attr_set[dev.index]) {
            cudaFuncSetAttribute(norm_rowwarp_vec_kernel<T, LAYER, PRE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 80 * 1024);
            attr_set[dev.index] = true;
        }
        const int64_t cap_vec = static_cast<int64_t>(dev.sm_count) * (smem > 56 * 1024 ? 2 : (smem > 36 * 1024 ? 4 : 6));
        if (blocks > cap_vec) blocks = cap_vec;
        norm_rowwarp_vec_kernel<T, LAYER, PRE><<<static_cast<unsigned>(blocks), kMaxThreads, smem, stream>>>(
            static_cast<const T*>(x), static_cast<const T*>(gamma), static_cast<const T*>(beta), static_cast<T*>(y), rows, cols, eps);
        count_launch();
        return launch_status();
    }
    norm_rowwarp_kernel<T, LAYER, PRE><<<static_cast<unsigned>(blocks), kMaxThreads, 0, stream>>>(
        static_cast<const T*>(x), static_cast<const T*>(gamma), static_cast<const T*>(beta), static_cast<T*>(y), rows,
        cols, eps);
    count_launch();
    return launch_status();
}

// LayerNorm(SiLU(x)) + gathered rows -> tokens, RMSNorm(tokens) -> normed: TMA-staged kernel only
template <typename T>
int token_tail_dispatch(const void* x, const void* gamma, const void* beta, void* tokens, int64_t rows, int cols,
                        float eps, const PostArgs& post, cudaStream_t stream) {
    const int N = Vec16<T>::N;
    const bool vec_ok = (cols % N == 0) && aligned16(x) && aligned16(tokens) && aligned16(gamma) && aligned16(beta) &&
                        aligned16(post.table_a) && (post.table_b == nullptr || aligned16(post.table_b)) &&
                        aligned16(post.gamma2) && aligned16(post.normed) && (cols / N) <= 256;
    if (!vec_ok) return TB200_ERR_UNSUPPORTED;
    const int chunks = cols / N;
    int G = 1;
    while (G < 32 && G < chunks) G <<= 1;
    const int cpl = (chunks + G - 1) / G;
    if (cpl <= 1) return launch_tma<T, true, 1, 4, kPreSilu, true>(x, gamma, beta, tokens, rows, cols, eps, G, stream, post);
    if (cpl <= 2) return launch_tma<T, true, 2, 2, kPreSilu, true>(x, gamma, beta, tokens, rows, cols, eps, G, stream, post);
    if (cpl <= 4) return launch_tma<T, true, 4, 1, kPreSilu, true>(x, gamma, beta, tokens, rows, cols, eps, G, stream, post);
    return launch_tma<T, true, 8, 1, kPreSilu, true>(x, gamma, beta, tokens, rows, cols, eps, G, stream, post);
}

template <bool LAYER, int PRE>
int norm_entry(const void* x, const void* gamma, const void* beta, void* y, int64_t rows, int32_t cols, float eps,
               int dtype, void* stream) {
    if (rows < 0 || cols < 1) return TB200_ERR_SHAPE;
    if (rows == 0) return TB200_OK;
    if (x == nullptr || gamma == nullptr || y == nullptr || ((LAYER || PRE == kPreBias) && beta == nullptr)) return TB200_ERR_NULL;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case TB200_F32: return norm_dispatch<float, LAYER, PRE>(x, gamma, beta, y, rows, cols, eps, s);
        case TB200_F16: return norm_dispatch<__half, LAYER, PRE>(x, gamma, beta, y, rows, cols, eps, s);
        case TB200_BF16: return norm_dispatch<__nv_bfloat16, LAYER, PRE>(x, gamma, beta, y, rows, cols, eps, s);
        default: return TB200_ERR_DTYPE;
    }
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_rmsnorm_fwd(const void* x, const void* gamma, void* y, int64_t rows, int32_t cols, float eps,
                                 int dtype, void* stream) {
    return tb200::norm_entry<false, tb200::kPreNone>(x, gamma, nullptr, y, rows, cols, eps, dtype, stream);
}

extern "C" int tb200_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, int64_t rows,
                                   int32_t cols, float eps, int dtype, void* stream) {
    return tb200::norm_entry<true, tb200::kPreNone>(x, gamma, beta, y, rows, cols, eps, dtype, stream);
}

extern "C" int tb200_rmsnorm_bias_fwd(const void* x, const void* in_bias, const void* gamma, void* y, int64_t rows,
                                      int32_t cols, float eps, int dtype, void* stream) {
    return tb200::norm_entry<false, tb200::kPreBias>(x, gamma, in_bias, y, rows, cols, eps, dtype, stream);
}

extern "C" int tb200_layernorm_silu_fwd(const void* x, const void* gamma, const void* beta, void* y, int64_t rows,
                                        int32_t cols, float eps, int dtype, void* stream) {
    return tb200::norm_entry<true, tb200::kPreSilu>(x, gamma, beta, y, rows, cols, eps, dtype, stream);
}

extern "C" int tb200_token_tail_select_fwd(const void* x, const void* ln_gamma, const void* ln_beta,
                                           const void* table_a, int64_t rows_a, const int64_t* ids_a,
                                           const void* table_b, int64_t rows_b, const int64_t* ids_b,
                                           const void* rms_gamma, const int32_t* row_dst, int64_t rows_out,
                                           void* tokens, void* normed, int64_t rows, int32_t cols, float ln_eps,
                                           float rms_eps, int dtype, void* stream) {
    using namespace tb200;
    if (rows < 0 || cols < 1 || rows_a < 1 || (table_b != nullptr && rows_b < 1)) return TB200_ERR_SHAPE;
    if (rows_a > INT32_MAX || (table_b != nullptr && rows_b > INT32_MAX)) return TB200_ERR_UNSUPPORTED;
    if (row_dst != nullptr && (rows_out < 0 || rows_out > INT32_MAX)) return TB200_ERR_SHAPE;
    if (rows == 0) return TB200_OK;
    if (x == nullptr || ln_gamma == nullptr || ln_beta == nullptr || table_a == nullptr || ids_a == nullptr ||
        (table_b != nullptr && ids_b == nullptr) || rms_gamma == nullptr || normed == nullptr ||
        (tokens == nullptr && !(row_dst != nullptr && rows_out == 0)))
        return TB200_ERR_NULL;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    PostArgs post{table_a, ids_a, rows_a, table_b, ids_b, rows_b, rms_gamma, normed, rms_eps, row_dst, rows_out};
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case TB200_F32: return token_tail_dispatch<float>(x, ln_gamma, ln_beta, tokens, rows, cols, ln_eps, post, s);
        case TB200_F16: return token_tail_dispatch<__half>(x, ln_gamma, ln_beta, tokens, rows, cols, ln_eps, post, s);
        case TB200_BF16: return token_tail_dispatch<__nv_bfloat16>(x, ln_gamma, ln_beta, tokens, rows, cols, ln_eps, post, s);
        default: return TB200_ERR_DTYPE;
    }
}

extern "C" int tb200_token_tail_fwd(const void* x, const void* ln_gamma, const void* ln_beta, const void* table_a,
                                    int64_t rows_a, const int64_t* ids_a, const void* table_b, int64_t rows_b,
                                    const int64_t* ids_b, const void* rms_gamma, void* tokens, void* normed,
                                    int64_t rows, int32_t cols, float ln_eps, float rms_eps, int dtype, void* stream) {
    return tb200_token_tail_select_fwd(x, ln_gamma, ln_beta, table_a, rows_a, ids_a, table_b, rows_b, ids_b, rms_gamma,
                                       nullptr, 0, tokens, normed, rows, cols, ln_eps, rms_eps, dtype, stream);
}
