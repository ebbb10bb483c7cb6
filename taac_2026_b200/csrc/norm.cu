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

constexpr int kThreads = 256;
constexpr int kStages = 4;
constexpr int kTileBytes = 16384;

template <typename T, bool LAYER, int CPL>
__global__ void __launch_bounds__(kThreads)
norm_tma_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta, T* __restrict__ y,
                int64_t rows, int cols, float eps, int rows_per_tile, int lanes_per_row, int* __restrict__ status) {
    constexpr int N = Vec16<T>::N;
    extern __shared__ __align__(128) uint8_t smem[];
    __shared__ uint64_t full_bar[kStages];

    const int tid = threadIdx.x;
    const int chunks = cols / N;  // 16-byte chunks per row
    const uint32_t row_bytes = static_cast<uint32_t>(chunks) * 16u;
    const uint32_t tile_bytes = row_bytes * static_cast<uint32_t>(rows_per_tile);
    const int64_t n_tiles = (rows + rows_per_tile - 1) / rows_per_tile;
    const int64_t first = blockIdx.x;
    const int64_t n_my = first < n_tiles ? (n_tiles - first + gridDim.x - 1) / gridDim.x : 0;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) mbar_init(&full_bar[s], 1);
        fence_mbar_init();
    }
    __syncthreads();

    auto tile_rows = [&](int64_t it) -> int {
        const int64_t r0 = (first + it * gridDim.x) * rows_per_tile;
        const int64_t left = rows - r0;
        return left < rows_per_tile ? static_cast<int>(left) : rows_per_tile;
    };
    auto issue_load = [&](int64_t it) {
        const int s = static_cast<int>(it % kStages);
        const int64_t r0 = (first + it * gridDim.x) * rows_per_tile;
        const uint32_t bytes = static_cast<uint32_t>(tile_rows(it)) * row_bytes;
        mbar_expect_tx(&full_bar[s], bytes);
        bulk_load(smem + static_cast<size_t>(s) * tile_bytes, reinterpret_cast<const uint8_t*>(x) + r0 * row_bytes,
                  bytes, &full_bar[s]);
    };

    if (tid == 0) {
        for (int64_t it = 0; it < n_my && it < kStages; ++it) issue_load(it);
    }

    const int G = lanes_per_row;
    const int group = tid / G;
    const int lane_g = tid % G;
    const int n_groups = kThreads / G;

    // gamma / beta for this lane's chunks stay in registers for the whole kernel
    float g[CPL][N];
    float b[CPL][N];
#pragma unroll
    for (int j = 0; j < CPL; ++j) {
        const int c = lane_g + j * G;
        if (c < chunks) {
            Vec16<T>::unpack(reinterpret_cast<const uint4*>(gamma)[c], g[j]);
            if (LAYER) Vec16<T>::unpack(reinterpret_cast<const uint4*>(beta)[c], b[j]);
        } else {
#pragma unroll
            for (int e = 0; e < N; ++e) {
                g[j][e] = 0.f;
                b[j][e] = 0.f;
            }
        }
    }
    const float inv_cols = 1.0f / static_cast<float>(cols);

    for (int64_t it = 0; it < n_my; ++it) {
        const int s = static_cast<int>(it % kStages);
        const uint32_t parity = static_cast<uint32_t>((it / kStages) & 1);
        const bool ok = mbar_wait(&full_bar[s], parity);
        if (__syncthreads_or(!ok)) {
            if (tid == 0 && status != nullptr) atomicExch(status, 1);
            break;
        }
        const int rows_here = tile_rows(it);
        uint4* tile = reinterpret_cast<uint4*>(smem + static_cast<size_t>(s) * tile_bytes);

        for (int r0 = 0; r0 < rows_here; r0 += n_groups) {
            const int r = r0 + group;
            const bool valid_row = r < rows_here;
            uint4* rowp = tile + static_cast<size_t>(valid_row ? r : 0) * chunks;
            float v[CPL][N];
            float sum = 0.f;
            float sq = 0.f;
#pragma unroll
            for (int j = 0; j < CPL; ++j) {
                const int c = lane_g + j * G;
                if (valid_row && c < chunks) {
                    Vec16<T>::unpack(rowp[c], v[j]);
                } else {
#pragma unroll
                    for (int e = 0; e < N; ++e) v[j][e] = 0.f;
                }
#pragma unroll
                for (int e = 0; e < N; ++e) {
                    if (LAYER) sum += v[j][e];
                    else sq = fmaf(v[j][e], v[j][e], sq);
                }
            }
            float mean = 0.f;
            if (LAYER) {
                for (int o = G >> 1; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
                mean = sum * inv_cols;
#pragma unroll
                for (int j = 0; j < CPL; ++j) {
                    const int c = lane_g + j * G;
                    if (c < chunks) {
#pragma unroll
                        for (int e = 0; e < N; ++e) {
                            const float d = v[j][e] - mean;
                            sq = fmaf(d, d, sq);
                        }
                    }
                }
            }
            for (int o = G >> 1; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
            const float inv = rsqrtf(sq * inv_cols + eps);
            if (valid_row) {
#pragma unroll
                for (int j = 0; j < CPL; ++j) {
                    const int c = lane_g + j * G;
                    if (c < chunks) {
                        float o[N];
#pragma unroll
                        for (int e = 0; e < N; ++e) {
                            if (LAYER) o[e] = fmaf((v[j][e] - mean) * inv, g[j][e], b[j][e]);
                            else o[e] = (v[j][e] * inv) * g[j][e];
                        }
                        rowp[c] = Vec16<T>::pack(o);
                    }
                }
            }
        }

        fence_proxy_async_smem();
        __syncthreads();
        if (tid == 0) {
            const int64_t r0g = (first + it * gridDim.x) * rows_per_tile;
            bulk_store(reinterpret_cast<uint8_t*>(y) + r0g * row_bytes, tile, static_cast<uint32_t>(rows_here) * row_bytes);
            bulk_commit();
            // The stage stored one iteration ago is free once its store has read shared memory.
            if (it >= 1 && it - 1 + kStages < n_my) {
                bulk_wait_read<1>();
                issue_load(it - 1 + kStages);
            }
        }
    }
    if (tid == 0) bulk_wait<0>();
}

// Warp per row, scalar accesses, any cols / alignment.
template <typename T, bool LAYER>
__global__ void __launch_bounds__(kThreads)
norm_rowwarp_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ beta,
                    T* __restrict__ y, int64_t rows, int cols, float eps) {
    const int lane = threadIdx.x & 31;
    const int64_t warp = (static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x) >> 5;
    const int64_t n_warps = (static_cast<int64_t>(gridDim.x) * kThreads) >> 5;
    const float inv_cols = 1.0f / static_cast<float>(cols);
    for (int64_t r = warp; r < rows; r += n_warps) {
        const T* xr = x + r * cols;
        T* yr = y + r * cols;
        float mean = 0.f;
        if (LAYER) {
            float sum = 0.f;
            for (int c = lane; c < cols; c += 32) sum += to_float<T>(xr[c]);
            for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            mean = sum * inv_cols;
        }
        float sq = 0.f;
        for (int c = lane; c < cols; c += 32) {
            const float d = to_float<T>(xr[c]) - mean;
            sq = fmaf(d, d, sq);
        }
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        const float inv = rsqrtf(sq * inv_cols + eps);
        for (int c = lane; c < cols; c += 32) {
            const float v = to_float<T>(xr[c]);
            float o;
            if (LAYER) o = fmaf((v - mean) * inv, to_float<T>(gamma[c]), to_float<T>(beta[c]));
            else o = (v * inv) * to_float<T>(gamma[c]);
            yr[c] = from_float<T>(o);
        }
    }
}

template <typename T, bool LAYER, int CPL>
int launch_tma(const void* x, const void* gamma, const void* beta, void* y, int64_t rows, int cols, float eps,
               int lanes_per_row, cudaStream_t stream) {
    const int N = Vec16<T>::N;
    const int chunks = cols / N;
    const int row_bytes = chunks * 16;
    const int n_groups = kThreads / lanes_per_row;
    int rows_per_tile = kTileBytes / row_bytes;
    if (rows_per_tile < 1) rows_per_tile = 1;
    // a whole number of passes over the row groups keeps every group busy
    if (rows_per_tile > n_groups) rows_per_tile -= rows_per_tile % n_groups;
    const size_t tile_bytes = static_cast<size_t>(rows_per_tile) * row_bytes;
    const size_t smem = tile_bytes * kStages;
    const DeviceInfo& dev = device_info();
    static bool attr_set = false;  // per instantiation; idempotent
    if (!attr_set) {
        cudaFuncSetAttribute(norm_tma_kernel<T, LAYER, CPL>, cudaFuncAttributeMaxDynamicSharedMemorySize, 96 * 1024);
        attr_set = true;
    }
    const int64_t n_tiles = (rows + rows_per_tile - 1) / rows_per_tile;
    int ctas_per_sm = static_cast<int>((200 * 1024) / (smem + 1024));
    if (ctas_per_sm > 4) ctas_per_sm = 4;
    if (ctas_per_sm < 1) ctas_per_sm = 1;
    int64_t grid = static_cast<int64_t>(dev.sm_count) * ctas_per_sm;
    if (grid > n_tiles) grid = n_tiles;
    if (grid < 1) grid = 1;
    norm_tma_kernel<T, LAYER, CPL><<<static_cast<unsigned>(grid), kThreads, smem, stream>>>(
        static_cast<const T*>(x), static_cast<const T*>(gamma), static_cast<const T*>(beta), static_cast<T*>(y), rows,
        cols, eps, rows_per_tile, lanes_per_row, nullptr);
    count_launch();
    return launch_status();
}

template <typename T, bool LAYER>
int norm_dispatch(const void* x, const void* gamma, const void* beta, void* y, int64_t rows, int cols, float eps,
                  cudaStream_t stream) {
    const int N = Vec16<T>::N;
    const bool vec_ok = (cols % N == 0) && aligned16(x) && aligned16(y) && aligned16(gamma) &&
                        (!LAYER || aligned16(beta)) && (cols / N) <= 256 && (cols / N) * 16 <= kTileBytes;
    if (vec_ok) {
        const int chunks = cols / N;
        int G = 1;
        while (G < 32 && G < chunks) G <<= 1;  // lanes per row: power of two, <= 32
        const int cpl = (chunks + G - 1) / G;
        if (cpl <= 1) return launch_tma<T, LAYER, 1>(x, gamma, beta, y, rows, cols, eps, G, stream);
        if (cpl <= 2) return launch_tma<T, LAYER, 2>(x, gamma, beta, y, rows, cols, eps, G, stream);
        if (cpl <= 4) return launch_tma<T, LAYER, 4>(x, gamma, beta, y, rows, cols, eps, G, stream);
        return launch_tma<T, LAYER, 8>(x, gamma, beta, y, rows, cols, eps, G, stream);
    }
    const DeviceInfo& dev = device_info();
    int64_t blocks = (rows + (kThreads / 32) - 1) / (kThreads / 32);
    const int64_t cap = static_cast<int64_t>(dev.sm_count) * 8;
    if (blocks > cap) blocks = cap;
    if (blocks < 1) blocks = 1;
    norm_rowwarp_kernel<T, LAYER><<<static_cast<unsigned>(blocks), kThreads, 0, stream>>>(
        static_cast<const T*>(x), static_cast<const T*>(gamma), static_cast<const T*>(beta), static_cast<T*>(y), rows,
        cols, eps);
    count_launch();
    return launch_status();
}

template <bool LAYER>
int norm_entry(const void* x, const void* gamma, const void* beta, void* y, int64_t rows, int32_t cols, float eps,
               int dtype, void* stream) {
    if (rows < 0 || cols < 1) return TB200_ERR_SHAPE;
    if (rows == 0) return TB200_OK;
    if (x == nullptr || gamma == nullptr || y == nullptr || (LAYER && beta == nullptr)) return TB200_ERR_NULL;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case TB200_F32: return norm_dispatch<float, LAYER>(x, gamma, beta, y, rows, cols, eps, s);
        case TB200_F16: return norm_dispatch<__half, LAYER>(x, gamma, beta, y, rows, cols, eps, s);
        case TB200_BF16: return norm_dispatch<__nv_bfloat16, LAYER>(x, gamma, beta, y, rows, cols, eps, s);
        default: return TB200_ERR_DTYPE;
    }
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_rmsnorm_fwd(const void* x, const void* gamma, void* y, int64_t rows, int32_t cols, float eps,
                                 int dtype, void* stream) {
    return tb200::norm_entry<false>(x, gamma, nullptr, y, rows, cols, eps, dtype, stream);
}

extern "C" int tb200_layernorm_fwd(const void* x, const void* gamma, const void* beta, void* y, int64_t rows,
                                   int32_t cols, float eps, int dtype, void* stream) {
    return tb200::norm_entry<true>(x, gamma, beta, y, rows, cols, eps, dtype, stream);
}
