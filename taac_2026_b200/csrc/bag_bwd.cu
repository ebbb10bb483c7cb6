// Sparse gradient of the bag-mean embedding lookup for sm_100a.
//
// Forward (tb200_bag_mean_fwd): out[b, :] = mean over the valid ids of bag b of table[id, :].  Its gradient with
// respect to the table touches only the looked-up rows, so it is handed on in the sparse (row list, value rows) form
// the reference builds for its sparse optimizer (`SparseEmbeddingBagMean.backward`,
// src/taac2026/infrastructure/modeling/embeddings.py:34-62; dense atomic-add form:
// accelerators/embedding/kernels/triton.py:105-151):
//     for every position (b, h):   rows[b * bag + h] = id,   vals[b * bag + h, :] = grad_out[b, :] / count_b
// with count_b the number of valid ids of the bag.  Positions whose id is padding (0) or outside the table keep the
// fixed layout: they name row 0 and carry zeros, which add nothing when the optimizer coalesces the list (the
// reference drops them instead; the coalesced gradients are equal).  No atomics: every output element is written by
// one thread, so the result does not depend on scheduling.
//
// HBM-bound: grad_out is read once per bag (its row stays in registers for all positions of the bag), vals is written
// once.  A group of lanes owns a bag: it counts the valid ids with a shuffle reduction, scales its 16-byte pieces of
// the gradient row once (true division, like the reference's `grad_out / counts`), and streams them out per position.
#include "tb200_common.cuh"

namespace tb200 {
void count_launch();

namespace {

template <typename T, typename IdT, int G>      // G lanes per bag (power of two), each with CPL 16-byte pieces of the row
__global__ void __launch_bounds__(256)
bag_mean_bwd_kernel(const IdT* __restrict__ ids, const T* __restrict__ grad_out, int64_t* __restrict__ rows_out,
                    T* __restrict__ vals_out, int64_t batch, int bag, int dim, int64_t vocab_rows) {
    constexpr int N = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const int sub = lane / G;
    const int lg = lane - sub * G;
    const int chunks = dim / N;
    const int64_t bags_per_block = (256 / 32) * (32 / G);
    // the loop bound is warp-uniform: the shuffles below name every lane of the warp
    for (int64_t base = (static_cast<int64_t>(blockIdx.x) * 8 + (threadIdx.x >> 5)) * (32 / G); base < batch;
         base += static_cast<int64_t>(gridDim.x) * bags_per_block) {
        const int64_t b = base + sub;
        const bool live = b < batch;
        int count = 0;
        for (int h = lg; h < bag; h += G) {
            const int64_t id = live ? static_cast<int64_t>(ids[b * bag + h]) : 0;
            count += (id > 0 && id < vocab_rows) ? 1 : 0;
        }
#pragma unroll
        for (int o = G >> 1; o > 0; o >>= 1) count += __shfl_xor_sync(0xffffffffu, count, o);
        const float denom = static_cast<float>(count > 0 ? count : 1);
        if (!live) continue;                               // no shuffle below this line
        for (int c = lg; c < chunks; c += G) {
            float g[N];
            Vec16<T>::unpack(*reinterpret_cast<const uint4*>(grad_out + b * dim + static_cast<int64_t>(c) * N), g);
#pragma unroll
            for (int e = 0; e < N; ++e) g[e] = __fdiv_rn(g[e], denom);
            const uint4 scaled = Vec16<T>::pack(g);
            const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
            for (int h = 0; h < bag; ++h) {
                const int64_t id = static_cast<int64_t>(ids[b * bag + h]);
                const bool valid = id > 0 && id < vocab_rows;
                *reinterpret_cast<uint4*>(vals_out + (b * bag + h) * dim + static_cast<int64_t>(c) * N) = valid ? scaled : zero;
                if (c == 0) rows_out[b * bag + h] = valid ? id : 0;
            }
        }
    }
}

template <typename T, typename IdT>
int launch(const void* ids, const void* grad_out, int64_t* rows_out, void* vals_out, int64_t batch, int bag, int dim,
           int64_t vocab_rows, cudaStream_t stream) {
    const int chunks = dim / Vec16<T>::N;
    int g = 1;
    while (g < chunks && g < 32) g <<= 1;
    const DeviceInfo& dev = device_info();
    const int64_t per_block = 8 * (32 / g);
    int64_t grid = (batch + per_block - 1) / per_block;
    const int64_t cap = static_cast<int64_t>(dev.sm_count) * 8;
    if (grid > cap) grid = cap;
#define TB200_BB(G_)                                                                                                       \
    bag_mean_bwd_kernel<T, IdT, G_><<<static_cast<unsigned>(grid), 256, 0, stream>>>(                                      \
        static_cast<const IdT*>(ids), static_cast<const T*>(grad_out), rows_out, static_cast<T*>(vals_out), batch, bag, dim, vocab_rows)
    switch (g) {
        case 1: TB200_BB(1); break;
        case 2: TB200_BB(2); break;
        case 4: TB200_BB(4); break;
        case 8: TB200_BB(8); break;
        case 16: TB200_BB(16); break;
        default: TB200_BB(32); break;
    }
#undef TB200_BB
    count_launch();
    return launch_status();
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_bag_mean_bwd(const void* ids, int ids_dtype, const void* grad_out, int64_t* rows_out, void* vals_out,
                                  int64_t batch, int32_t bag, int32_t dim, int64_t vocab_rows, int dtype, void* stream) {
    using namespace tb200;
    if (batch < 0 || bag < 1 || dim < 1 || vocab_rows < 1) return TB200_ERR_SHAPE;
    const int esize = dtype_size(dtype);
    if (esize == 0 || (ids_dtype != TB200_I32 && ids_dtype != TB200_I64)) return TB200_ERR_DTYPE;
    if (dim % (16 / esize) != 0) return TB200_ERR_ALIGN;
    if (batch == 0) return TB200_OK;
    if (ids == nullptr || grad_out == nullptr || rows_out == nullptr || vals_out == nullptr) return TB200_ERR_NULL;
    if (!aligned16(grad_out) || !aligned16(vals_out)) return TB200_ERR_ALIGN;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define TB200_DISPATCH(T_)                                                                                                  \
    return ids_dtype == TB200_I32 ? launch<T_, int32_t>(ids, grad_out, rows_out, vals_out, batch, bag, dim, vocab_rows, s)  \
                                  : launch<T_, int64_t>(ids, grad_out, rows_out, vals_out, batch, bag, dim, vocab_rows, s)
    switch (dtype) {
        case TB200_F32: TB200_DISPATCH(float);
        case TB200_F16: TB200_DISPATCH(__half);
        default: TB200_DISPATCH(__nv_bfloat16);
    }
#undef TB200_DISPATCH
}
