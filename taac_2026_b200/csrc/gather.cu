// Sparse-field embedding gather and bag-mean pooling for sm_100a.
//
// HBM-bound random row reads.  Each CTA first stages the ids of its block of output rows
// in shared memory (coalesced reads of the int32/int64 id matrix, clamp applied once),
// then sub-warp groups of lanes move table rows with 128-bit loads/stores, several rows
// in flight per group.  Pooling accumulates in fp32 in hot order and divides once by the
// number of valid ids with an IEEE division, which makes a bag of one id an exact copy.
#include "tb200_common.cuh"

namespace tb200 {
void count_launch();

namespace {

constexpr int kThreads = 256;
constexpr int kRowsPerCta = 512;   // gather: ids staged per CTA
constexpr int kMaxStagedIds = 8192;  // bag-mean: ids staged per CTA (int32)

__device__ __forceinline__ uint4 ld_nc_v4(const uint4* p) {
    uint4 v;
    asm volatile("ld.global.nc.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ void st_cs_v4(uint4* p, const uint4& v) {
    asm volatile("st.global.cs.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w)
                 : "memory");
}

template <typename I>
__device__ __forceinline__ int64_t load_id(const void* ids, int64_t idx) {
    return static_cast<int64_t>(static_cast<const I*>(ids)[idx]);
}

// ---------------------------------------------------------------------------------------
// gather_rows: out[i, col0 : col0 + dim] = table[clamp(ids[...]), :]
// ---------------------------------------------------------------------------------------
template <typename I>
__global__ void __launch_bounds__(kThreads)
gather_rows_kernel(const uint4* __restrict__ table, int64_t vocab_rows, int chunks, const void* __restrict__ ids,
                   int64_t n, int64_t seq_len, int64_t ids_batch_stride, uint4* __restrict__ out,
                   int64_t out_stride_chunks, int out_col0_chunks, int lanes_per_row) {
    __shared__ int32_t ids_s[kRowsPerCta];
    const int tid = threadIdx.x;
    const int64_t base = static_cast<int64_t>(blockIdx.x) * kRowsPerCta;
    const int here = static_cast<int>(n - base < kRowsPerCta ? n - base : kRowsPerCta);
    for (int j = tid; j < here; j += kThreads) {
        const int64_t i = base + j;
        const int64_t b = i / seq_len;
        const int64_t l = i - b * seq_len;
        int64_t id = load_id<I>(ids, b * ids_batch_stride + l);
        id = id < 0 ? 0 : (id > vocab_rows - 1 ? vocab_rows - 1 : id);
        ids_s[j] = static_cast<int32_t>(id);
    }
    __syncthreads();

    const int G = lanes_per_row;
    const int group = tid / G;
    const int lane_g = tid % G;
    const int n_groups = kThreads / G;
    constexpr int U = 4;  // rows in flight per group
    for (int j0 = group * U; j0 < here; j0 += n_groups * U) {
        for (int c = lane_g; c < chunks; c += G) {
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int j = j0 + u;
                if (j < here) v[u] = ld_nc_v4(table + static_cast<int64_t>(ids_s[j]) * chunks + c);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int j = j0 + u;
                if (j < here) st_cs_v4(out + (base + j) * out_stride_chunks + out_col0_chunks + c, v[u]);
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// bag-mean over one table or over the tables of many fields
// ---------------------------------------------------------------------------------------
struct BagArgs {
    const void* const* tables;  // [n_fields] or nullptr -> table0
    const int64_t* rows;        // [n_fields]
    const int32_t* offsets;     // [n_fields]
    const int32_t* lengths;     // [n_fields]
    const void* table0;
    int64_t rows0;
    int32_t n_fields;
    int32_t max_bag;
    int32_t ids_cols;
    int32_t clamp;  // 1: clamp ids into the table (field bank); 0: ids outside (0, rows) are skipped
    int32_t bags_per_cta;
    int32_t chunks;
    int32_t lanes_per_row;
    int64_t n_bags;  // batch * n_fields
    const uint8_t* missing;     // [batch, missing_cols] flags or nullptr: out += missing_rows[field] where set
    const void* missing_rows;   // [n_fields, dim]
    int32_t missing_cols;
};

template <typename T, typename I>
__global__ void __launch_bounds__(kThreads)
bag_mean_kernel(BagArgs a, const void* __restrict__ ids, T* __restrict__ out) {
    constexpr int N = Vec16<T>::N;
    extern __shared__ int32_t bag_ids[];  // [bags_per_cta, max_bag]; 0 = skip
    const int tid = threadIdx.x;
    const int64_t q_base = static_cast<int64_t>(blockIdx.x) * a.bags_per_cta;
    const int here = static_cast<int>(a.n_bags - q_base < a.bags_per_cta ? a.n_bags - q_base : a.bags_per_cta);

    for (int j = tid; j < here * a.max_bag; j += kThreads) {
        const int ql = j / a.max_bag;
        const int h = j - ql * a.max_bag;
        const int64_t q = q_base + ql;
        const int64_t bidx = q / a.n_fields;
        const int f = static_cast<int>(q - bidx * a.n_fields);
        int64_t vrows = a.rows0;
        int off = 0;
        int len = a.max_bag;
        if (a.tables != nullptr) {
            vrows = a.rows[f];
            off = a.offsets[f];
            len = a.lengths[f];
        }
        int64_t id = 0;
        if (h < len) {
            id = load_id<I>(ids, bidx * a.ids_cols + off + h);
            if (a.clamp) id = id < 0 ? 0 : (id > vrows - 1 ? vrows - 1 : id);
            else if (id < 0 || id >= vrows) id = 0;
        }
        bag_ids[j] = static_cast<int32_t>(id);
    }
    __syncthreads();

    const int G = a.lanes_per_row;
    const int group = tid / G;
    const int lane_g = tid % G;
    const int n_groups = kThreads / G;
    const int chunks = a.chunks;
    constexpr int U = 4;  // table rows in flight per lane

    if (a.max_bag == 1) {
        // One id per bag (the field bank of single-valued features): the pooled row is the table row itself, so a lane
        // group keeps the rows of four bags in flight instead of walking one bag after the other.
        constexpr int B4 = 4;
        for (int ql0 = group; ql0 < here; ql0 += B4 * n_groups) {
            for (int c = lane_g; c < chunks; c += G) {
                uint4 v[B4];
                int id[B4];
#pragma unroll
                for (int u = 0; u < B4; ++u) {
                    const int ql = ql0 + u * n_groups;
                    id[u] = ql < here ? bag_ids[ql] : 0;
                    v[u] = make_uint4(0, 0, 0, 0);
                    if (id[u] != 0) {
                        const int64_t q = q_base + ql;
                        const uint4* table = a.tables != nullptr ? static_cast<const uint4*>(a.tables[q % a.n_fields])
                                                                 : static_cast<const uint4*>(a.table0);
                        v[u] = ld_nc_v4(table + static_cast<int64_t>(id[u]) * chunks + c);
                    }
                }
#pragma unroll
                for (int u = 0; u < B4; ++u) {
                    const int ql = ql0 + u * n_groups;
                    if (ql >= here) continue;
                    const int64_t q = q_base + ql;
                    uint4 o = v[u];
                    if (a.missing != nullptr) {
                        const int64_t bidx = q / a.n_fields;
                        const int f = static_cast<int>(q - bidx * a.n_fields);
                        if (a.missing[bidx * a.missing_cols + f] != 0) {
                            float x[N], m[N];
                            Vec16<T>::unpack(o, x);
                            Vec16<T>::unpack(static_cast<const uint4*>(a.missing_rows)[f * chunks + c], m);
#pragma unroll
                            for (int e = 0; e < N; ++e) x[e] += m[e];
                            o = Vec16<T>::pack(x);
                        }
                    }
                    st_cs_v4(reinterpret_cast<uint4*>(out) + q * chunks + c, o);
                }
            }
        }
        return;
    }

    for (int ql = group; ql < here; ql += n_groups) {
        const int64_t q = q_base + ql;
        const uint4* table = static_cast<const uint4*>(a.table0);
        if (a.tables != nullptr) table = static_cast<const uint4*>(a.tables[q % a.n_fields]);
        const int32_t* my_ids = bag_ids + ql * a.max_bag;
        int count = 0;
        for (int h = 0; h < a.max_bag; ++h) count += my_ids[h] != 0;
        for (int c = lane_g; c < chunks; c += G) {
            float acc[N];
#pragma unroll
            for (int e = 0; e < N; ++e) acc[e] = 0.f;
            uint4 first = make_uint4(0, 0, 0, 0);
            for (int h0 = 0; h0 < a.max_bag; h0 += U) {
                uint4 v[U];
                int id[U];
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    id[u] = (h0 + u < a.max_bag) ? my_ids[h0 + u] : 0;
                    if (id[u] != 0) v[u] = ld_nc_v4(table + static_cast<int64_t>(id[u]) * chunks + c);
                }
#pragma unroll
                for (int u = 0; u < U; ++u) {
                    if (id[u] != 0) {
                        first = v[u];
                        float f[N];
                        Vec16<T>::unpack(v[u], f);
#pragma unroll
                        for (int e = 0; e < N; ++e) acc[e] += f[e];
                    }
                }
            }
            uint4 o;
            if (count == 1) {
                o = first;  // a single valid id: the row itself, bit for bit
            } else if (count == 0) {
                o = make_uint4(0, 0, 0, 0);
            } else {
                const float denom = static_cast<float>(count);
#pragma unroll
                for (int e = 0; e < N; ++e) acc[e] = __fdiv_rn(acc[e], denom);
                o = Vec16<T>::pack(acc);
            }
            if (a.missing != nullptr) {
                // the per-field "missing" row, added to the pooled row as stored (one rounding for the mean, one
                // for the sum: what `pooled + mask[..., None] * missing_embeddings` gives as two tensor operations)
                const int64_t bidx = q / a.n_fields;
                const int f = static_cast<int>(q - bidx * a.n_fields);
                if (a.missing[bidx * a.missing_cols + f] != 0) {
                    float x[N], m[N];
                    Vec16<T>::unpack(o, x);
                    Vec16<T>::unpack(static_cast<const uint4*>(a.missing_rows)[f * chunks + c], m);
#pragma unroll
                    for (int e = 0; e < N; ++e) x[e] += m[e];
                    o = Vec16<T>::pack(x);
                }
            }
            st_cs_v4(reinterpret_cast<uint4*>(out) + q * chunks + c, o);
        }
    }
}

// ---------------------------------------------------------------------------------------
// scatter_rows: dst[ids[i], :] = src[i, :] (+ bias[i / rows_per_group, :]) (+ residual[ids[i], :])
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
scatter_rows_kernel(uint4* __restrict__ dst, int64_t dst_stride_chunks, int dst_col0_chunks,
                    const int64_t* __restrict__ ids, const uint4* __restrict__ src, int chunks, int64_t n,
                    const uint4* __restrict__ bias, int64_t rows_per_group, const uint4* __restrict__ residual,
                    int64_t res_stride_chunks, int lanes_per_row) {
    constexpr int N = Vec16<T>::N;
    const int G = lanes_per_row;
    const int group = threadIdx.x / G;
    const int lane_g = threadIdx.x % G;
    const int n_groups = kThreads / G;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * n_groups + group; i < n; i += static_cast<int64_t>(gridDim.x) * n_groups) {
        const int64_t row = ids[i];
        const uint4* brow = bias != nullptr ? bias + (i / rows_per_group) * chunks : nullptr;
        for (int c = lane_g; c < chunks; c += G) {
            uint4 v = ld_nc_v4(src + i * chunks + c);
            if (brow != nullptr || residual != nullptr) {
                float f[N];
                Vec16<T>::unpack(v, f);
                if (brow != nullptr) {
                    float b[N];
                    Vec16<T>::unpack(brow[c], b);
#pragma unroll
                    for (int e = 0; e < N; ++e) f[e] += b[e];
                }
                if (residual != nullptr) {
                    float r[N];
                    Vec16<T>::unpack(residual[row * res_stride_chunks + c], r);
#pragma unroll
                    for (int e = 0; e < N; ++e) f[e] += r[e];
                }
                v = Vec16<T>::pack(f);
            }
            dst[row * dst_stride_chunks + dst_col0_chunks + c] = v;
        }
    }
}


// ---------------------------------------------------------------------------------------
// add_gathered_rows: x[i, :] = x[i, :] + table_a[ids_a[i], :]  (then + table_b[ids_b[i], :]), in place.
// Each sum is rounded to T before the next one, like two separate tensor additions.
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
add_gathered_rows_kernel(uint4* __restrict__ x, int64_t n, int chunks, const uint4* __restrict__ table_a, int64_t rows_a,
                         const int64_t* __restrict__ ids_a, const uint4* __restrict__ table_b, int64_t rows_b,
                         const int64_t* __restrict__ ids_b, int lanes_per_row) {
    constexpr int N = Vec16<T>::N;
    const int G = lanes_per_row;
    const int group = threadIdx.x / G;
    const int lane_g = threadIdx.x % G;
    const int n_groups = kThreads / G;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * n_groups + group; i < n; i += static_cast<int64_t>(gridDim.x) * n_groups) {
        int64_t ia = ids_a[i];
        ia = ia < 0 ? 0 : (ia > rows_a - 1 ? rows_a - 1 : ia);
        int64_t ib = 0;
        if (table_b != nullptr) {
            ib = ids_b[i];
            ib = ib < 0 ? 0 : (ib > rows_b - 1 ? rows_b - 1 : ib);
        }
        for (int c = lane_g; c < chunks; c += G) {
            float f[N], a[N];
            Vec16<T>::unpack(x[i * chunks + c], f);
            Vec16<T>::unpack(ld_nc_v4(table_a + ia * chunks + c), a);
#pragma unroll
            for (int e = 0; e < N; ++e) f[e] += a[e];
            uint4 v = Vec16<T>::pack(f);
            if (table_b != nullptr) {
                Vec16<T>::unpack(v, f);   // the first sum as T stores it
                Vec16<T>::unpack(ld_nc_v4(table_b + ib * chunks + c), a);
#pragma unroll
                for (int e = 0; e < N; ++e) f[e] += a[e];
                v = Vec16<T>::pack(f);
            }
            x[i * chunks + c] = v;
        }
    }
}

// ---------------------------------------------------------------------------------------
// bias_act_rows: x[r, :] = act(x[r, :] + bias[r / rows_per_group, :]), in place, act = identity or SiLU; the
// sum is rounded to T before the activation, like an addition followed by a separate SiLU.
// ---------------------------------------------------------------------------------------
template <typename T, bool SILU>
__global__ void __launch_bounds__(kThreads)
bias_act_rows_kernel(uint4* __restrict__ x, int64_t rows, int chunks, const uint4* __restrict__ bias,
                     int64_t rows_per_group) {
    constexpr int N = Vec16<T>::N;
    constexpr int U = 4;   // 16-byte pieces in flight per thread
    // a thread keeps one column piece c and walks down the rows, so its bias piece changes only with the group
    const int cols_per_cta = kThreads < chunks ? kThreads : chunks;       // pieces of a row served by one CTA pass
    const int rows_per_pass = kThreads / cols_per_cta;
    const int c0 = threadIdx.x % cols_per_cta;
    const int r_in = threadIdx.x / cols_per_cta;
    if (r_in >= rows_per_pass) return;
    for (int c = c0; c < chunks; c += cols_per_cta) {
        for (int64_t r = static_cast<int64_t>(blockIdx.x) * rows_per_pass * U + r_in; r < rows;
             r += static_cast<int64_t>(gridDim.x) * rows_per_pass * U) {
            uint4 v[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t ru = r + static_cast<int64_t>(u) * rows_per_pass;
                if (ru < rows) v[u] = x[ru * chunks + c];
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int64_t ru = r + static_cast<int64_t>(u) * rows_per_pass;
                if (ru >= rows) continue;
                float f[N], b[N];
                Vec16<T>::unpack(v[u], f);
                Vec16<T>::unpack(bias[(ru / rows_per_group) * chunks + c], b);
#pragma unroll
                for (int e = 0; e < N; ++e) f[e] += b[e];
                if (SILU) {
                    Vec16<T>::unpack(Vec16<T>::pack(f), f);
#pragma unroll
                    for (int e = 0; e < N; ++e) f[e] = __fdividef(f[e], 1.0f + __expf(-f[e]));
                }
                x[ru * chunks + c] = Vec16<T>::pack(f);
            }
        }
    }
}


int lanes_for(int chunks) {
    int g = 1;
    while (g < 32 && g < chunks) g <<= 1;
    return g;
}

template <typename T>
int bag_launch(BagArgs a, const void* ids, int ids_dtype, void* out, cudaStream_t stream) {
    int per = kMaxStagedIds / a.max_bag;
    if (per < 1) return TB200_ERR_UNSUPPORTED;
    if (per > 256) per = 256;
    a.bags_per_cta = per;
    a.lanes_per_row = lanes_for(a.chunks);
    const int64_t grid = (a.n_bags + per - 1) / per;
    if (grid > 0x7FFFFFFFll) return TB200_ERR_SHAPE;
    const size_t smem = static_cast<size_t>(per) * a.max_bag * sizeof(int32_t);
    if (ids_dtype == TB200_I64)
        bag_mean_kernel<T, int64_t><<<static_cast<unsigned>(grid), kThreads, smem, stream>>>(a, ids, static_cast<T*>(out));
    else
        bag_mean_kernel<T, int32_t><<<static_cast<unsigned>(grid), kThreads, smem, stream>>>(a, ids, static_cast<T*>(out));
    count_launch();
    return launch_status();
}

int bag_entry(BagArgs a, int32_t dim, const void* ids, int ids_dtype, int64_t batch, void* out, int dtype,
              void* stream) {
    if (batch < 0 || dim < 1 || a.max_bag < 0 || a.n_fields < 1) return TB200_ERR_SHAPE;
    if (batch == 0) return TB200_OK;
    if (ids_dtype != TB200_I32 && ids_dtype != TB200_I64) return TB200_ERR_DTYPE;
    const int es = dtype_size(dtype);
    if (es == 0) return TB200_ERR_DTYPE;
    if (out == nullptr || (a.max_bag > 0 && ids == nullptr)) return TB200_ERR_NULL;
    if ((static_cast<int64_t>(dim) * es) % 16 != 0 || !aligned16(out)) return TB200_ERR_ALIGN;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    a.chunks = dim * es / 16;
    a.n_bags = batch * a.n_fields;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (a.max_bag == 0 && a.missing == nullptr) {  // every bag is empty
        cudaError_t e = cudaMemsetAsync(out, 0, static_cast<size_t>(a.n_bags) * dim * es, s);
        return e == cudaSuccess ? TB200_OK : static_cast<int>(e);
    }
    if (a.max_bag == 0) return TB200_ERR_UNSUPPORTED;
    switch (dtype) {
        case TB200_F32: return bag_launch<float>(a, ids, ids_dtype, out, s);
        case TB200_F16: return bag_launch<__half>(a, ids, ids_dtype, out, s);
        case TB200_BF16: return bag_launch<__nv_bfloat16>(a, ids, ids_dtype, out, s);
        default: return TB200_ERR_DTYPE;
    }
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_bag_mean_fwd(const void* table, int64_t vocab_rows, int32_t dim, const void* ids, int ids_dtype,
                                  int64_t batch, int32_t bag, void* out, int dtype, void* stream) {
    using namespace tb200;
    if (table == nullptr) return TB200_ERR_NULL;
    if (vocab_rows < 1 || vocab_rows > 0x7FFFFFFFll) return TB200_ERR_SHAPE;
    if (!aligned16(table)) return TB200_ERR_ALIGN;
    BagArgs a{};
    a.tables = nullptr;
    a.table0 = table;
    a.rows0 = vocab_rows;
    a.n_fields = 1;
    a.max_bag = bag;
    a.ids_cols = bag;
    a.clamp = 0;
    return bag_entry(a, dim, ids, ids_dtype, batch, out, dtype, stream);
}

extern "C" int tb200_fields_bag_mean_fwd(const void* const* tables, const int64_t* rows, const int32_t* offsets,
                                         const int32_t* lengths, int32_t n_fields, int32_t max_bag, int32_t dim,
                                         const void* ids, int ids_dtype, int64_t batch, int32_t ids_cols, void* out,
                                         int dtype, void* stream) {
    using namespace tb200;
    if (tables == nullptr || rows == nullptr || offsets == nullptr || lengths == nullptr) return TB200_ERR_NULL;
    BagArgs a{};
    a.tables = tables;
    a.rows = rows;
    a.offsets = offsets;
    a.lengths = lengths;
    a.n_fields = n_fields;
    a.max_bag = max_bag;
    a.ids_cols = ids_cols;
    a.clamp = 1;
    return bag_entry(a, dim, ids, ids_dtype, batch, out, dtype, stream);
}

extern "C" int tb200_fields_bag_mean_missing_fwd(const void* const* tables, const int64_t* rows, const int32_t* offsets,
                                                 const int32_t* lengths, int32_t n_fields, int32_t max_bag, int32_t dim,
                                                 const void* ids, int ids_dtype, int64_t batch, int32_t ids_cols,
                                                 const uint8_t* missing, int32_t missing_cols, const void* missing_rows,
                                                 void* out, int dtype, void* stream) {
    using namespace tb200;
    if (tables == nullptr || rows == nullptr || offsets == nullptr || lengths == nullptr) return TB200_ERR_NULL;
    if (missing == nullptr || missing_rows == nullptr) return TB200_ERR_NULL;
    if (missing_cols < n_fields) return TB200_ERR_SHAPE;
    if (!aligned16(missing_rows)) return TB200_ERR_ALIGN;
    BagArgs a{};
    a.tables = tables;
    a.rows = rows;
    a.offsets = offsets;
    a.lengths = lengths;
    a.n_fields = n_fields;
    a.max_bag = max_bag;
    a.ids_cols = ids_cols;
    a.clamp = 1;
    a.missing = missing;
    a.missing_rows = missing_rows;
    a.missing_cols = missing_cols;
    return bag_entry(a, dim, ids, ids_dtype, batch, out, dtype, stream);
}

extern "C" int tb200_gather_rows(const void* table, int64_t vocab_rows, int32_t dim, const void* ids, int ids_dtype,
                                 int64_t n, int64_t seq_len, int64_t ids_batch_stride, void* out, int64_t out_stride,
                                 int32_t out_col0, int dtype, void* stream) {
    using namespace tb200;
    if (n < 0 || dim < 1 || seq_len < 1 || out_stride < dim || out_col0 < 0) return TB200_ERR_SHAPE;
    if (vocab_rows < 1 || vocab_rows > 0x7FFFFFFFll) return TB200_ERR_SHAPE;
    if (n == 0) return TB200_OK;
    if (ids_dtype != TB200_I32 && ids_dtype != TB200_I64) return TB200_ERR_DTYPE;
    const int es = dtype_size(dtype);
    if (es == 0) return TB200_ERR_DTYPE;
    if (table == nullptr || ids == nullptr || out == nullptr) return TB200_ERR_NULL;
    if ((static_cast<int64_t>(dim) * es) % 16 != 0 || (out_stride * es) % 16 != 0 ||
        (static_cast<int64_t>(out_col0) * es) % 16 != 0 || !aligned16(table) || !aligned16(out))
        return TB200_ERR_ALIGN;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    const int chunks = dim * es / 16;
    const int64_t grid = (n + kRowsPerCta - 1) / kRowsPerCta;
    if (grid > 0x7FFFFFFFll) return TB200_ERR_SHAPE;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int G = lanes_for(chunks);
    if (ids_dtype == TB200_I64)
        gather_rows_kernel<int64_t><<<static_cast<unsigned>(grid), kThreads, 0, s>>>(
            static_cast<const uint4*>(table), vocab_rows, chunks, ids, n, seq_len, ids_batch_stride,
            static_cast<uint4*>(out), out_stride * es / 16, out_col0 * es / 16, G);
    else
        gather_rows_kernel<int32_t><<<static_cast<unsigned>(grid), kThreads, 0, s>>>(
            static_cast<const uint4*>(table), vocab_rows, chunks, ids, n, seq_len, ids_batch_stride,
            static_cast<uint4*>(out), out_stride * es / 16, out_col0 * es / 16, G);
    count_launch();
    return launch_status();
}

extern "C" int tb200_scatter_rows(void* dst, int64_t dst_rows, int64_t dst_stride, int32_t dst_col0, const int64_t* ids,
                                  const void* src, int64_t n, int32_t dim, const void* bias, int64_t rows_per_group,
                                  const void* residual, int64_t residual_stride, int dtype, void* stream) {
    using namespace tb200;
    if (n < 0 || dim < 1 || dst_rows < 0 || dst_stride < dim || dst_col0 < 0 || dst_col0 + dim > dst_stride) return TB200_ERR_SHAPE;
    if (bias != nullptr && rows_per_group < 1) return TB200_ERR_SHAPE;
    if (residual != nullptr && residual_stride < dim) return TB200_ERR_SHAPE;
    if (n == 0) return TB200_OK;
    const int es = dtype_size(dtype);
    if (es == 0) return TB200_ERR_DTYPE;
    if (dst == nullptr || ids == nullptr || src == nullptr) return TB200_ERR_NULL;
    if ((static_cast<int64_t>(dim) * es) % 16 != 0 || (dst_stride * es) % 16 != 0 || (static_cast<int64_t>(dst_col0) * es) % 16 != 0 ||
        (residual != nullptr && (residual_stride * es) % 16 != 0) || !aligned16(dst) || !aligned16(src) ||
        (bias != nullptr && !aligned16(bias)) || (residual != nullptr && !aligned16(residual)))
        return TB200_ERR_ALIGN;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    const int chunks = dim * es / 16;
    const int G = lanes_for(chunks);
    const int n_groups = kThreads / G;
    int64_t grid = (n + n_groups - 1) / n_groups;
    const int64_t cap = static_cast<int64_t>(device_info().sm_count) * 16;
    if (grid > cap) grid = cap;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define TB200_SCATTER(T)                                                                                              \
    scatter_rows_kernel<T><<<static_cast<unsigned>(grid), kThreads, 0, s>>>(                                          \
        static_cast<uint4*>(dst), dst_stride * es / 16, dst_col0 * es / 16, ids, static_cast<const uint4*>(src), chunks, \
        n, static_cast<const uint4*>(bias), rows_per_group < 1 ? 1 : rows_per_group, static_cast<const uint4*>(residual), \
        residual_stride * es / 16, G)
    switch (dtype) {
        case TB200_F32: TB200_SCATTER(float); break;
        case TB200_F16: TB200_SCATTER(__half); break;
        case TB200_BF16: TB200_SCATTER(__nv_bfloat16); break;
        default: return TB200_ERR_DTYPE;
    }
#undef TB200_SCATTER
    count_launch();
    return launch_status();
}

extern "C" int tb200_add_gathered_rows(void* x, int64_t n, int32_t dim, const void* table_a, int64_t rows_a,
                                       const int64_t* ids_a, const void* table_b, int64_t rows_b, const int64_t* ids_b,
                                       int dtype, void* stream) {
    using namespace tb200;
    if (n < 0 || dim < 1 || rows_a < 1 || (table_b != nullptr && rows_b < 1)) return TB200_ERR_SHAPE;
    if (n == 0) return TB200_OK;
    const int es = dtype_size(dtype);
    if (es == 0) return TB200_ERR_DTYPE;
    if (x == nullptr || table_a == nullptr || ids_a == nullptr || (table_b != nullptr && ids_b == nullptr)) return TB200_ERR_NULL;
    if ((static_cast<int64_t>(dim) * es) % 16 != 0 || !aligned16(x) || !aligned16(table_a) ||
        (table_b != nullptr && !aligned16(table_b)))
        return TB200_ERR_ALIGN;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    const int chunks = dim * es / 16;
    const int G = lanes_for(chunks);
    const int n_groups = kThreads / G;
    int64_t grid = (n + n_groups - 1) / n_groups;
    const int64_t cap = static_cast<int64_t>(device_info().sm_count) * 16;
    if (grid > cap) grid = cap;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define TB200_ADDG(T)                                                                                                 \
    add_gathered_rows_kernel<T><<<static_cast<unsigned>(grid), kThreads, 0, s>>>(                                     \
        static_cast<uint4*>(x), n, chunks, static_cast<const uint4*>(table_a), rows_a, ids_a,                         \
        static_cast<const uint4*>(table_b), rows_b, ids_b, G)
    switch (dtype) {
        case TB200_F32: TB200_ADDG(float); break;
        case TB200_F16: TB200_ADDG(__half); break;
        case TB200_BF16: TB200_ADDG(__nv_bfloat16); break;
        default: return TB200_ERR_DTYPE;
    }
#undef TB200_ADDG
    count_launch();
    return launch_status();
}

extern "C" int tb200_bias_act_rows(void* x, int64_t rows, int32_t cols, const void* bias, int64_t rows_per_group,
                                   int32_t act, int dtype, void* stream) {
    using namespace tb200;
    if (rows < 0 || cols < 1 || rows_per_group < 1) return TB200_ERR_SHAPE;
    if (act != 0 && act != 1) return TB200_ERR_UNSUPPORTED;
    if (rows == 0) return TB200_OK;
    const int es = dtype_size(dtype);
    if (es == 0) return TB200_ERR_DTYPE;
    if (x == nullptr || bias == nullptr) return TB200_ERR_NULL;
    if ((static_cast<int64_t>(cols) * es) % 16 != 0 || !aligned16(x) || !aligned16(bias)) return TB200_ERR_ALIGN;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    const int chunks = cols * es / 16;
    const int rows_per_pass = chunks >= kThreads ? 1 : kThreads / chunks;
    int64_t grid = (rows + rows_per_pass * 4 - 1) / (rows_per_pass * 4);
    const int64_t cap = static_cast<int64_t>(device_info().sm_count) * 16;
    if (grid > cap) grid = cap;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
#define TB200_BSILU(T)                                                                                        \
    if (act == 1)                                                                                             \
        bias_act_rows_kernel<T, true><<<static_cast<unsigned>(grid), kThreads, 0, s>>>(                       \
            static_cast<uint4*>(x), rows, chunks, static_cast<const uint4*>(bias), rows_per_group);           \
    else                                                                                                      \
        bias_act_rows_kernel<T, false><<<static_cast<unsigned>(grid), kThreads, 0, s>>>(                      \
            static_cast<uint4*>(x), rows, chunks, static_cast<const uint4*>(bias), rows_per_group)
    switch (dtype) {
        case TB200_F32: TB200_BSILU(float); break;
        case TB200_F16: TB200_BSILU(__half); break;
        case TB200_BF16: TB200_BSILU(__nv_bfloat16); break;
        default: return TB200_ERR_DTYPE;
    }
#undef TB200_BSILU
    count_launch();
    return launch_status();
}
