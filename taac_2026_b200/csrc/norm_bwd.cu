// RMSNorm / LayerNorm backward for sm_100a (the first training-side kernels of the path).
//
//   RMSNorm    y = x r w,            r = rsqrt(mean(x^2) + eps)
//              g = dy w;   dx = r g - x r^3 mean(g x);                  dw = sum_rows dy x r
//   LayerNorm  y = xh w + b,         xh = (x - mu) rs,  rs = rsqrt(var + eps)
//              g = dy w;   dx = rs (g - mean(g) - xh mean(g xh));       dw = sum_rows dy xh,  db = sum_rows dy
//
// These are the gradients of the reference's accelerated norms
// (src/taac2026/infrastructure/accelerators/normalization/kernels/triton.py:83-116 RMSNorm backward, :277-320 LayerNorm
// backward: dX per row plus per-block partial dW / dB that a second step reduces).  The statistics are recomputed from
// x (the forward kernels keep nothing), in fp32.
//
// HBM-bound: x and dy are read once, dx is written once (3 rows * cols * esize bytes per call).  A group of G lanes
// (G = the row's 16-byte pieces, at most 32) owns a row; a lane keeps its pieces of x and dy in registers, the row
// sums are shuffle reductions inside the group, and the lane adds its columns' dw / db terms to fp32 accumulators that
// live across all rows the lane sees.  At the end of a CTA the accumulators of lanes that own the same columns are
// summed in a fixed order (shuffles across the groups of a warp, then the warps through shared memory), and the CTA
// writes one row of partial sums; a second small kernel adds the partial rows, again in a fixed order, so the result
// does not depend on scheduling.
#include "tb200_common.cuh"

namespace tb200 {
void count_launch();

namespace {

constexpr int kWarps = 8;
constexpr int kThreads = kWarps * 32;
constexpr int kMaxPartials = 592;   // CTAs of the main kernel = rows of the partial table (4 per SM on 148 SMs)

template <typename T>
__device__ __forceinline__ uint4 ld_stream(const T* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// CPL: 16-byte pieces of a row per lane; G: lanes per row (power of two); LAYER: LayerNorm, else RMSNorm
template <typename T, int CPL, int G, bool LAYER>
__global__ void __launch_bounds__(kThreads)
norm_bwd_kernel(const T* __restrict__ x, const T* __restrict__ gamma, const T* __restrict__ dy, T* __restrict__ dx,
                float* __restrict__ partial_w, float* __restrict__ partial_b, int64_t rows, int cols, float eps) {
    constexpr int N = Vec16<T>::N;           // elements per 16-byte piece
    constexpr int RPW = 32 / G;              // rows a warp handles at a time
    extern __shared__ float red[];           // [kWarps][cols] (x 2 for LayerNorm)
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int sub = lane / G;                // which of the warp's rows
    const int lg = lane - sub * G;           // lane inside the row's group
    const int chunks = cols / N;
    const float inv_cols = 1.0f / static_cast<float>(cols);

    float gm[CPL][N];
    float aw[CPL][N], ab[LAYER ? CPL : 1][N];
#pragma unroll
    for (int j = 0; j < CPL; ++j) {
        const int c = lg + j * G;
#pragma unroll
        for (int e = 0; e < N; ++e) {
            gm[j][e] = 0.f;
            aw[j][e] = 0.f;
            if (LAYER) ab[j][e] = 0.f;
        }
        if (c < chunks) Vec16<T>::unpack(*reinterpret_cast<const uint4*>(gamma + static_cast<int64_t>(c) * N), gm[j]);
    }

    // The loop bound is the same for every lane of a warp (the shuffles below name all 32 lanes); a lane whose row
    // lies past the end works on zeros and stores nothing.
    const int64_t row_step = static_cast<int64_t>(gridDim.x) * kWarps * RPW;
    // The pieces of the NEXT row of this lane group are requested before the current row is worked on, so that every
    // warp always has loads in flight under its shuffle chains (a zero piece stands for "past the end").
    uint4 nx[CPL], ng[CPL];
    auto fetch = [&](int64_t row) {
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
            const int c = lg + j * G;
            if (row < rows && c < chunks) {
                nx[j] = ld_stream(x + row * cols + static_cast<int64_t>(c) * N);
                ng[j] = ld_stream(dy + row * cols + static_cast<int64_t>(c) * N);
            } else {
                nx[j] = ng[j] = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    };
    const int64_t first = (static_cast<int64_t>(blockIdx.x) * kWarps + warp) * RPW;
    fetch(first + sub);
    for (int64_t base = first; base < rows; base += row_step) {
        const int64_t row = base + sub;
        const bool live = row < rows;
        float xv[CPL][N], gv[CPL][N];
        float s1 = 0.f, s2 = 0.f;            // RMS: s2 = sum x^2;  Layer: s1 = sum x, s2 = centred sum of squares
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
            Vec16<T>::unpack(nx[j], xv[j]);
            Vec16<T>::unpack(ng[j], gv[j]);
        }
        fetch(row + row_step);
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
#pragma unroll
            for (int e = 0; e < N; ++e) {
                if (LAYER) s1 += xv[j][e];
                else s2 = fmaf(xv[j][e], xv[j][e], s2);
            }
        }
        float mean = 0.f;
        if (LAYER) {
#pragma unroll
            for (int o = G >> 1; o > 0; o >>= 1) s1 += __shfl_xor_sync(0xffffffffu, s1, o);
            mean = s1 * inv_cols;
#pragma unroll
            for (int j = 0; j < CPL; ++j) {
                const int c = lg + j * G;
#pragma unroll
                for (int e = 0; e < N; ++e) {
                    xv[j][e] = c < chunks ? xv[j][e] - mean : 0.f;       // keep the centred value
                    s2 = fmaf(xv[j][e], xv[j][e], s2);
                }
            }
        }
#pragma unroll
        for (int o = G >> 1; o > 0; o >>= 1) s2 += __shfl_xor_sync(0xffffffffu, s2, o);
        const float r = rsqrtf(s2 * inv_cols + eps);
        // xh = x r (RMS) or (x - mu) rs (Layer); the dw / db terms of this row; g = dy w; row sums of g and g xh
        float sg = 0.f, sgx = 0.f;
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
#pragma unroll
            for (int e = 0; e < N; ++e) {
                const float xh = xv[j][e] * r;
                aw[j][e] = fmaf(gv[j][e], xh, aw[j][e]);
                if (LAYER) ab[j][e] += gv[j][e];
                const float g = gv[j][e] * gm[j][e];
                if (LAYER) sg += g;
                sgx = fmaf(g, xh, sgx);
                xv[j][e] = xh;
                gv[j][e] = g;
            }
        }
#pragma unroll
        for (int o = G >> 1; o > 0; o >>= 1) {
            sgx += __shfl_xor_sync(0xffffffffu, sgx, o);
            if (LAYER) sg += __shfl_xor_sync(0xffffffffu, sg, o);
        }
        const float mg = sg * inv_cols, mgx = sgx * inv_cols;
#pragma unroll
        for (int j = 0; j < CPL; ++j) {
            const int c = lg + j * G;
            if (live && c < chunks) {
                float o[N];
#pragma unroll
                for (int e = 0; e < N; ++e) o[e] = r * (gv[j][e] - mg - xv[j][e] * mgx);     // mg = 0 for RMSNorm
                *reinterpret_cast<uint4*>(dx + row * cols + static_cast<int64_t>(c) * N) = Vec16<T>::pack(o);
            }
        }
    }

    // ---- the CTA's partial sums of dw (and db), in a fixed order: groups of a warp, then warps
#pragma unroll
    for (int j = 0; j < CPL; ++j) {
#pragma unroll
        for (int e = 0; e < N; ++e) {
#pragma unroll
            for (int o = 16; o >= G; o >>= 1) {
                aw[j][e] += __shfl_xor_sync(0xffffffffu, aw[j][e], o);
                if (LAYER) ab[j][e] += __shfl_xor_sync(0xffffffffu, ab[j][e], o);
            }
        }
        const int c = lg + j * G;
        if (sub == 0 && c < chunks) {
#pragma unroll
            for (int e = 0; e < N; ++e) {
                red[warp * cols + c * N + e] = aw[j][e];
                if (LAYER) red[(kWarps + warp) * cols + c * N + e] = ab[j][e];
            }
        }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < cols; i += kThreads) {
        float w = 0.f, b = 0.f;
#pragma unroll
        for (int k = 0; k < kWarps; ++k) {
            w += red[k * cols + i];
            if (LAYER) b += red[(kWarps + k) * cols + i];
        }
        partial_w[static_cast<int64_t>(blockIdx.x) * cols + i] = w;
        if (LAYER) partial_b[static_cast<int64_t>(blockIdx.x) * cols + i] = b;
    }
}

// dgamma[i] = sum over the partial rows, rounded to T; the same for dbeta.  A block owns 32 columns: thread (ty, tx)
// adds the partial rows ty, ty + 32, ... of column tx (coalesced across tx), thread (0, tx) then adds the 32 sums in
// the order of ty.  The order is fixed, so the result does not depend on scheduling; one thread per column walking
// all ~600 partial rows was a chain of dependent loads that cost 25-30 us per call whatever the width.
template <typename T>
__global__ void __launch_bounds__(1024)
norm_bwd_reduce_kernel(const float* __restrict__ partial_w, const float* __restrict__ partial_b, T* __restrict__ dgamma,
                       T* __restrict__ dbeta, int n_partials, int cols) {
    __shared__ float sw[32][33], sb[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int i = blockIdx.x * 32 + tx;
    float w = 0.f, b = 0.f;
    if (i < cols) {
        for (int p = ty; p < n_partials; p += 32) {
            w += partial_w[static_cast<int64_t>(p) * cols + i];
            if (partial_b != nullptr) b += partial_b[static_cast<int64_t>(p) * cols + i];
        }
    }
    sw[ty][tx] = w;
    sb[ty][tx] = b;
    __syncthreads();
    if (ty == 0 && i < cols) {
        float ws = 0.f, bs = 0.f;
#pragma unroll
        for (int k = 0; k < 32; ++k) {
            ws += sw[k][tx];
            bs += sb[k][tx];
        }
        dgamma[i] = from_float<T>(ws);
        if (dbeta != nullptr) dbeta[i] = from_float<T>(bs);
    }
}

int grid_for(int64_t rows, int rows_per_cta) {
    const DeviceInfo& dev = device_info();
    int64_t ctas = (rows + rows_per_cta - 1) / rows_per_cta;
    const int64_t cap = dev.valid ? static_cast<int64_t>(dev.sm_count) * 4 : kMaxPartials;
    if (ctas > cap) ctas = cap;
    if (ctas > kMaxPartials) ctas = kMaxPartials;
    return ctas < 1 ? 1 : static_cast<int>(ctas);
}

template <typename T, int CPL, int G, bool LAYER>
int launch_one(const void* x, const void* gamma, const void* dy, void* dx, float* pw, float* pb, int64_t rows, int cols, float eps,
               int grid, cudaStream_t stream) {
    const size_t smem = static_cast<size_t>(kWarps) * cols * sizeof(float) * (LAYER ? 2 : 1);
    static bool attr_set[64] = {};
    const DeviceInfo& dev = device_info();
    if (!attr_set[dev.index]) {
        cudaFuncSetAttribute(norm_bwd_kernel<T, CPL, G, LAYER>, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * kWarps * 1024 * static_cast<int>(sizeof(float)));
        attr_set[dev.index] = true;
    }
    norm_bwd_kernel<T, CPL, G, LAYER><<<grid, kThreads, smem, stream>>>(
        static_cast<const T*>(x), static_cast<const T*>(gamma), static_cast<const T*>(dy), static_cast<T*>(dx), pw, pb, rows, cols, eps);
    count_launch();
    return launch_status();
}

// chunks = 16-byte pieces per row: G = the next power of two up to 32, CPL = pieces per lane
template <typename T, bool LAYER>
int launch_shape(const void* x, const void* gamma, const void* dy, void* dx, float* pw, float* pb, int64_t rows, int cols, float eps,
                 int* grid_out, cudaStream_t stream) {
    const int chunks = cols / Vec16<T>::N;
    int g = 1;
    while (g < chunks && g < 32) g <<= 1;
    const int cpl = (chunks + g - 1) / g;
    const int grid = grid_for(rows, kWarps * (32 / g));
    *grid_out = grid;
#define TB200_NB(CPL_, G_) return launch_one<T, CPL_, G_, LAYER>(x, gamma, dy, dx, pw, pb, rows, cols, eps, grid, stream)
    if (g < 32) {
        switch (g) {
            case 1: TB200_NB(1, 1);
            case 2: TB200_NB(1, 2);
            case 4: TB200_NB(1, 4);
            case 8: TB200_NB(1, 8);
            default: TB200_NB(1, 16);
        }
    }
    switch (cpl) {
        case 1: TB200_NB(1, 32);
        case 2: TB200_NB(2, 32);
        case 3: TB200_NB(3, 32);
        case 4: TB200_NB(4, 32);
        default: return TB200_ERR_UNSUPPORTED;
    }
#undef TB200_NB
}

template <bool LAYER>
int norm_bwd(const void* x, const void* gamma, const void* dy, void* dx, void* dgamma, void* dbeta, float* workspace,
             int64_t rows, int32_t cols, float eps, int dtype, void* stream) {
    if (rows < 0 || cols < 1) return TB200_ERR_SHAPE;
    const int esize = dtype_size(dtype);
    if (esize == 0) return TB200_ERR_DTYPE;
    const int per16 = 16 / esize;
    if (cols % per16 != 0 || cols / per16 > 128) return TB200_ERR_UNSUPPORTED;   // whole 16-byte pieces, at most four per lane
    if (x == nullptr || gamma == nullptr || dy == nullptr || dx == nullptr || dgamma == nullptr || workspace == nullptr ||
        (LAYER && dbeta == nullptr))
        return TB200_ERR_NULL;
    if (!aligned16(x) || !aligned16(gamma) || !aligned16(dy) || !aligned16(dx)) return TB200_ERR_ALIGN;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    float* pw = workspace;
    float* pb = LAYER ? workspace + static_cast<size_t>(kMaxPartials) * cols : nullptr;
    int grid = 1;
    int code = TB200_OK;
    if (rows == 0) {
        grid = 0;
    } else {
        switch (dtype) {
            case TB200_F32: code = launch_shape<float, LAYER>(x, gamma, dy, dx, pw, pb, rows, cols, eps, &grid, s); break;
            case TB200_F16: code = launch_shape<__half, LAYER>(x, gamma, dy, dx, pw, pb, rows, cols, eps, &grid, s); break;
            default: code = launch_shape<__nv_bfloat16, LAYER>(x, gamma, dy, dx, pw, pb, rows, cols, eps, &grid, s); break;
        }
        if (code != TB200_OK) return code;
    }
    const int rgrid = (cols + 31) / 32;
    switch (dtype) {
        case TB200_F32:
            norm_bwd_reduce_kernel<float><<<rgrid, 1024, 0, s>>>(pw, pb, static_cast<float*>(dgamma), static_cast<float*>(dbeta), grid, cols);
            break;
        case TB200_F16:
            norm_bwd_reduce_kernel<__half><<<rgrid, 1024, 0, s>>>(pw, pb, static_cast<__half*>(dgamma), static_cast<__half*>(dbeta), grid, cols);
            break;
        default:
            norm_bwd_reduce_kernel<__nv_bfloat16><<<rgrid, 1024, 0, s>>>(pw, pb, static_cast<__nv_bfloat16*>(dgamma),
                                                                          static_cast<__nv_bfloat16*>(dbeta), grid, cols);
            break;
    }
    count_launch();
    return launch_status();
}

}  // namespace
}  // namespace tb200

extern "C" int64_t tb200_norm_bwd_workspace_bytes(int32_t cols, int32_t layer_norm) {
    if (cols < 1) return 0;
    return static_cast<int64_t>(tb200::kMaxPartials) * cols * static_cast<int64_t>(sizeof(float)) * (layer_norm ? 2 : 1);
}

extern "C" int tb200_rmsnorm_bwd(const void* x, const void* gamma, const void* dy, void* dx, void* dgamma, float* workspace,
                                 int64_t rows, int32_t cols, float eps, int dtype, void* stream) {
    return tb200::norm_bwd<false>(x, gamma, dy, dx, dgamma, nullptr, workspace, rows, cols, eps, dtype, stream);
}

extern "C" int tb200_layernorm_bwd(const void* x, const void* gamma, const void* dy, void* dx, void* dgamma, void* dbeta,
                                   float* workspace, int64_t rows, int32_t cols, float eps, int dtype, void* stream) {
    return tb200::norm_bwd<true>(x, gamma, dy, dx, dgamma, dbeta, workspace, rows, cols, eps, dtype, stream);
}
