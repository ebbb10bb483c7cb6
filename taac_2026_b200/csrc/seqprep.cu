// Integer preprocessing of a behaviour-sequence domain, one CTA per sample:
//   * duplicate-event removal (keep the LAST occurrence of every distinct active event, in order), and
//   * the six sequence statistics,
// which the reference computes with F stable argsorts plus gather / scatter passes over [B, L] int64
// tensors.  Here every sample is handled in shared memory: the active events are inserted into an
// open-addressing hash table keyed by the full feature tuple (exact comparison against the slot's
// representative event, so hash collisions cannot merge different events), each slot remembers the
// largest position that hit it, and an event survives iff it is that position.  A block-wide scan
// then compacts the survivors.  All arithmetic is integer; the statistics are converted to fp32 the
// same way the reference converts them.
#include "tb200_common.cuh"

namespace tb200 {
void count_launch();

namespace {

constexpr int kThreads = 256;
constexpr int kEdges = 63;

__constant__ int64_t c_edges[kEdges] = {
    5, 10, 15, 20, 25, 30, 35, 40, 45, 50, 55, 60, 120, 180, 240, 300, 360, 420, 480, 540, 600, 900, 1200, 1500, 1800,
    2100, 2400, 2700, 3000, 3300, 3600, 5400, 7200, 9000, 10800, 12600, 14400, 16200, 18000, 19800, 21600, 32400,
    43200, 54000, 64800, 75600, 86400, 172800, 259200, 345600, 432000, 518400, 604800, 1123200, 1641600, 2160000,
    2592000, 4320000, 6048000, 7776000, 11664000, 15552000, 31536000};

// number of edges strictly below gap (torch.searchsorted, side = "left"), clamped as the reference does
__device__ __forceinline__ int gap_bucket(int64_t ts, int64_t request) {
    if (ts == 0) return 0;
    int64_t gap = request - ts;
    if (gap < 0) gap = 0;
    int lo = 0, hi = kEdges;
    while (lo < hi) {
        const int mid = (lo + hi) >> 1;
        if (c_edges[mid] < gap) lo = mid + 1;
        else hi = mid;
    }
    return (lo > kEdges - 1 ? kEdges - 1 : lo) + 1;
}

__device__ __forceinline__ uint32_t mix(uint64_t x) {
    x ^= x >> 33;
    x *= 0xff51afd7ed558ccdULL;
    x ^= x >> 33;
    x *= 0xc4ceb9fe1a85ec53ULL;
    x ^= x >> 33;
    return static_cast<uint32_t>(x);
}

__global__ void __launch_bounds__(kThreads)
seqprep_kernel(const int64_t* __restrict__ values, const int64_t* __restrict__ lengths,
               const int64_t* __restrict__ timestamps, const int64_t* __restrict__ request_ts, int n_feat, int max_len,
               int table_size, int64_t* __restrict__ out_len, int32_t* __restrict__ out_src,
               float* __restrict__ out_stats) {
    extern __shared__ int32_t smem_i[];
    int32_t* rep = smem_i;                    // [table_size] representative position of the slot, -1 = empty
    int32_t* last = rep + table_size;         // [table_size] largest position that hit the slot
    int32_t* slot_of = last + table_size;     // [max_len] slot of every active position, -1 = inactive
    int32_t* scan = slot_of + max_len;        // [kThreads] block scan scratch
    __shared__ int s_active, s_positive, s_kept;

    const int b = blockIdx.x;
    const int tid = threadIdx.x;
    const int64_t* row = values + static_cast<int64_t>(b) * n_feat * max_len;
    int64_t raw = lengths[b];
    raw = raw < 0 ? 0 : (raw > max_len ? max_len : raw);
    const int raw_len = static_cast<int>(raw);

    for (int i = tid; i < table_size; i += kThreads) {
        rep[i] = -1;
        last[i] = -1;
    }
    if (tid == 0) {
        s_active = 0;
        s_positive = 0;
        s_kept = 0;
    }
    __syncthreads();

    // ---- insert the active events
    int n_active = 0, n_positive = 0;
    for (int p = tid; p < max_len; p += kThreads) {
        bool any_pos = false;
        uint64_t h = 0x9e3779b97f4a7c15ULL;
        for (int f = 0; f < n_feat; ++f) {
            const int64_t v = row[static_cast<int64_t>(f) * max_len + p];
            if (v > 0) {
                any_pos = true;
                ++n_positive;
            }
            h = (h ^ static_cast<uint64_t>(v)) * 0x100000001b3ULL + (h >> 29);
        }
        int my_slot = -1;
        if (any_pos && p < raw_len) {
            ++n_active;
            uint32_t s = mix(h) & (table_size - 1);
            for (int probe = 0; probe < table_size; ++probe) {
                const int cur = atomicCAS(&rep[s], -1, p);
                bool same = cur == -1 || cur == p;
                if (!same) {
                    same = true;
                    for (int f = 0; f < n_feat; ++f)
                        if (row[static_cast<int64_t>(f) * max_len + cur] != row[static_cast<int64_t>(f) * max_len + p]) {
                            same = false;
                            break;
                        }
                }
                if (same) {
                    atomicMax(&last[s], p);
                    my_slot = static_cast<int>(s);
                    break;
                }
                s = (s + 1) & (table_size - 1);
            }
        }
        slot_of[p] = my_slot;
    }
    atomicAdd(&s_active, n_active);
    atomicAdd(&s_positive, n_positive);
    __syncthreads();

    // ---- survivors, compacted in original order (chunks of kThreads positions, running offset)
    int32_t* src_row = out_src + static_cast<int64_t>(b) * max_len;
    int base = 0;
    for (int p0 = 0; p0 < max_len; p0 += kThreads) {
        const int p = p0 + tid;
        const bool keep = p < max_len && slot_of[p] >= 0 && last[slot_of[p]] == p;
        scan[tid] = keep ? 1 : 0;
        __syncthreads();
        for (int off = 1; off < kThreads; off <<= 1) {  // Hillis-Steele inclusive scan
            const int add = tid >= off ? scan[tid - off] : 0;
            __syncthreads();
            scan[tid] += add;
            __syncthreads();
        }
        if (keep) src_row[base + scan[tid] - 1] = p;
        base += scan[kThreads - 1];
        __syncthreads();
    }
    if (tid == 0) s_kept = base;
    __syncthreads();
    const int kept = s_kept;
    const bool changed = kept != raw_len && raw_len > 1;
    if (!changed) {  // untouched rows keep every position, active or not
        for (int p = tid; p < max_len; p += kThreads) src_row[p] = p;
    } else {
        for (int p = kept + tid; p < max_len; p += kThreads) src_row[p] = -1;  // zero-filled tail
    }
    if (tid == 0) {
        out_len[b] = changed ? static_cast<int64_t>(kept) : lengths[b];
        float* st = out_stats + static_cast<int64_t>(b) * 6;
        const int active = s_active;
        const bool has = active > 0;
        const float active_f = static_cast<float>(active);
        const float kept_f = static_cast<float>(kept);
        const int64_t denom = static_cast<int64_t>(raw_len) * n_feat > 1 ? static_cast<int64_t>(raw_len) * n_feat : 1;
        st[0] = has ? static_cast<float>(raw_len) : 0.f;
        st[1] = has ? active_f : 0.f;
        st[2] = has ? kept_f : 0.f;
        st[3] = has ? 1.0f - __fdiv_rn(kept_f, fmaxf(active_f, 1.0f)) : 0.f;
        st[4] = has ? __fdiv_rn(static_cast<float>(s_positive), static_cast<float>(denom)) : 0.f;
        const int last_index = raw_len > 0 ? raw_len - 1 : 0;
        st[5] = (has && raw_len > 0) ? static_cast<float>(gap_bucket(timestamps[static_cast<int64_t>(b) * max_len + last_index], request_ts[b])) : 0.f;
    }
}

// ------------------------------------------------------------------------------------------------
// Index vectors of the packed token matrix.  Sample b owns rows [cu_rows[b], cu_rows[b + 1]): first its
// seq_count[b] sequence tokens, then its non-sequence tokens.  Sequence token j is the event at input position
// src[b, start[b] + j] (start = first position the tail crop keeps); this kernel looks up, for every row, the
// feature ids (hashed into buckets where a table is a compressed one), the position j and the time-gap bucket;
// rows of non-sequence tokens get zeros (the padding rows of the tables).  One CTA per sample.
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(128)
token_index_kernel(const int64_t* __restrict__ values, const int64_t* __restrict__ timestamps,
                   const int64_t* __restrict__ request_ts, const int32_t* __restrict__ src,
                   const int64_t* __restrict__ cu_rows, const int64_t* __restrict__ seq_count,
                   const int64_t* __restrict__ start, const int64_t* __restrict__ edges, int n_edges,
                   const int64_t* __restrict__ hash_buckets, int n_feat, int max_len, int64_t total_rows,
                   int64_t* __restrict__ ids_out, int64_t* __restrict__ pos_out, int64_t* __restrict__ bucket_out) {
    const int64_t b = blockIdx.x;
    const int64_t row0 = cu_rows[b];
    const int64_t n_rows = cu_rows[b + 1] - row0;
    const int64_t n_seq = seq_count[b];
    const int64_t first = start[b];
    const int64_t req = request_ts[b];
    for (int64_t j = threadIdx.x; j < n_rows; j += blockDim.x) {
        const int64_t row = row0 + j;
        int64_t p = -1;
        if (j < n_seq && first + j < max_len) p = src[b * max_len + first + j];
        const bool live = p >= 0 && p < max_len;
        for (int f = 0; f < n_feat; ++f) {
            const int64_t buckets = hash_buckets[f];
            if (buckets < 0) continue;                       // feature without a table: nothing to write
            int64_t v = live ? values[(b * n_feat + f) * max_len + p] : 0;
            if (buckets > 0) v = v > 0 ? (v - 1) % buckets + 1 : 0;
            ids_out[static_cast<int64_t>(f) * total_rows + row] = v;
        }
        pos_out[row] = live ? j : 0;
        if (bucket_out != nullptr) {
            int64_t bucket = 0;
            if (live) {
                const int64_t t = timestamps[b * max_len + p];
                if (t != 0) {
                    int64_t gap = req - t;
                    if (gap < 0) gap = 0;
                    int lo = 0, hi = n_edges;                  // number of edges < gap
                    while (lo < hi) {
                        const int mid = (lo + hi) >> 1;
                        if (edges[mid] < gap) lo = mid + 1;
                        else hi = mid;
                    }
                    bucket = (lo < n_edges - 1 ? lo : n_edges - 1) + 1;
                }
            }
            bucket_out[row] = bucket;
        }
    }
}

// ---------------------------------------------------------------------------------------
// Row plan of the packed layout.  The pyramid schedule (padded widths S[0..L], experiments/onetrans/model.py:317-348)
// is static; what depends on the batch is how many valid sequence tokens every sample still has at each layer:
//     raw = clamp(len[b], 0, max_len)      start[b] = max(raw - S[0], 0)      n0[b] = min(raw, S[0])
//     counts[l][b] = max(n0[b] - (S[0] - S[l]), 0)            rows[l][b] = counts[l][b] + ns
//     cu[l] = exclusive prefix sum of rows[l]   (B + 1 entries, as int64 and as int32)
//     meta[l] = (sum_b rows[l][b], max_b rows[l][b])          ns_rows0[b][j] = cu[0][b] + counts[0][b] + j
// One CTA per layer: a thread owns one sample of a 1024-sample tile (coalesced reads), the tile's rows go through a
// block scan (warp shuffles + one shared array of warp totals) and the running total is carried from tile to tile.
// It replaces some ninety one-line tensor operations per batch.
// ---------------------------------------------------------------------------------------
constexpr int kPlanThreads = 1024;
constexpr int kPlanMaxLayers = 64;

struct PlanWidths {
    int32_t w[kPlanMaxLayers + 1];
};

__global__ void __launch_bounds__(kPlanThreads)
pyramid_plan_kernel(const int64_t* __restrict__ lengths, int batch, int max_len, PlanWidths widths, int ns,
                    int64_t* __restrict__ start, int64_t* __restrict__ n0_out, int64_t* __restrict__ counts,
                    int64_t* __restrict__ cu, int32_t* __restrict__ cu32, int64_t* __restrict__ meta,
                    int64_t* __restrict__ ns_rows0) {
    __shared__ int64_t warp_sum[32];
    __shared__ int64_t warp_max[32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int l = blockIdx.x;
    const int width = widths.w[0];
    const int64_t drop = width - widths.w[l];
    int64_t* cu_l = cu + static_cast<int64_t>(l) * (batch + 1);
    int32_t* cu32_l = cu32 + static_cast<int64_t>(l) * (batch + 1);
    int64_t running = 0, mx = 0;
    for (int tile = 0; tile < batch; tile += kPlanThreads) {
        const int b = tile + tid;
        int64_t c = 0, r = 0;
        if (b < batch) {
            const int64_t len = lengths[b];
            const int64_t raw = len < 0 ? 0 : (len > max_len ? max_len : len);
            const int64_t n0 = raw < width ? raw : width;
            c = n0 > drop ? n0 - drop : 0;
            r = c + ns;
            counts[static_cast<int64_t>(l) * batch + b] = c;
            if (l == 0) {
                start[b] = raw > width ? raw - width : 0;
                n0_out[b] = n0;
            }
        }
        mx = max(mx, r);
        int64_t incl = r;                                   // inclusive scan inside the warp
#pragma unroll
        for (int o = 1; o < 32; o <<= 1) {
            const int64_t up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        if (lane == 31) warp_sum[warp] = incl;
        __syncthreads();
        int64_t before = 0, tile_total = 0;
        for (int w = 0; w < 32; ++w) {                      // 32 shared-memory reads, same address per warp: broadcasts
            const int64_t v = warp_sum[w];
            before += w < warp ? v : 0;
            tile_total += v;
        }
        const int64_t first_row = running + before + incl - r;
        if (b < batch) {
            cu_l[b] = first_row;
            cu32_l[b] = static_cast<int32_t>(first_row);
            if (l == 0)
                for (int j = 0; j < ns; ++j) ns_rows0[static_cast<int64_t>(b) * ns + j] = first_row + c + j;
        }
        running += tile_total;
        __syncthreads();                                    // warp_sum is rewritten by the next tile
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = max(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    if (lane == 0) warp_max[warp] = mx;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < 32; ++w) mx = max(mx, warp_max[w]);
        cu_l[batch] = running;
        cu32_l[batch] = static_cast<int32_t>(running);
        meta[2 * l] = running;
        meta[2 * l + 1] = mx;
    }
}

// Rows of layer l that the pyramid keeps for layer l + 1 (the last rows of every sample), in the next layer's order:
//     src[cu1[b] + r] = cu0[b] + (counts0[b] - counts1[b]) + r            r < counts1[b] + ns
//     ns_rows1[b][j] = cu1[b] + counts1[b] + j
//     row_dst[cu0[b] + i] = i < dropped ? -1 : cu1[b] + i - dropped        (optional: destination of every row of l)
__global__ void __launch_bounds__(128)
pyramid_kept_rows_kernel(const int64_t* __restrict__ cu0, const int64_t* __restrict__ cu1, const int64_t* __restrict__ counts0,
                         const int64_t* __restrict__ counts1, int ns, int64_t* __restrict__ src, int64_t* __restrict__ ns_rows1,
                         int32_t* __restrict__ row_dst) {
    const int b = blockIdx.x;
    const int64_t base0 = cu0[b], base1 = cu1[b];
    const int64_t c0 = counts0[b], c1 = counts1[b];
    const int64_t dropped = c0 - c1;
    const int64_t rows1 = c1 + ns;
    for (int64_t r = threadIdx.x; r < rows1; r += blockDim.x) src[base1 + r] = base0 + dropped + r;
    for (int j = threadIdx.x; j < ns; j += blockDim.x) ns_rows1[static_cast<int64_t>(b) * ns + j] = base1 + c1 + j;
    if (row_dst != nullptr) {
        const int64_t rows0 = c0 + ns;
        for (int64_t i = threadIdx.x; i < rows0; i += blockDim.x)
            row_dst[base0 + i] = i < dropped ? -1 : static_cast<int32_t>(base1 + i - dropped);
    }
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_pyramid_plan(const int64_t* lengths, int32_t batch, int32_t max_len, const int32_t* widths,
                                  int32_t n_layers, int32_t ns, int64_t* start, int64_t* n0, int64_t* counts, int64_t* cu,
                                  int32_t* cu32, int64_t* meta, int64_t* ns_rows0, void* stream) {
    using namespace tb200;
    if (batch < 0 || max_len < 0 || n_layers < 0 || n_layers > kPlanMaxLayers || ns < 0) return TB200_ERR_SHAPE;
    if (widths == nullptr || start == nullptr || n0 == nullptr || counts == nullptr || cu == nullptr || cu32 == nullptr ||
        meta == nullptr || (batch > 0 && lengths == nullptr) || (ns > 0 && batch > 0 && ns_rows0 == nullptr))
        return TB200_ERR_NULL;
    PlanWidths w{};
    for (int l = 0; l <= n_layers; ++l) {
        if (widths[l] < 0 || widths[l] > widths[0]) return TB200_ERR_SHAPE;
        w.w[l] = widths[l];
    }
    // the int32 offsets must hold the largest total: every sample at most widths[0] + ns rows
    if ((static_cast<int64_t>(widths[0]) + ns) * batch > 0x7FFFFFFFll) return TB200_ERR_SHAPE;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    pyramid_plan_kernel<<<static_cast<unsigned>(n_layers + 1), kPlanThreads, 0, static_cast<cudaStream_t>(stream)>>>(
        lengths, batch, max_len, w, ns, start, n0, counts, cu, cu32, meta, ns_rows0);
    count_launch();
    return launch_status();
}

extern "C" int tb200_pyramid_kept_rows(const int64_t* cu0, const int64_t* cu1, const int64_t* counts0, const int64_t* counts1,
                                       int32_t batch, int32_t ns, int64_t* src, int64_t* ns_rows1, int32_t* row_dst,
                                       void* stream) {
    using namespace tb200;
    if (batch < 0 || ns < 0) return TB200_ERR_SHAPE;
    if (batch == 0) return TB200_OK;
    if (cu0 == nullptr || cu1 == nullptr || counts0 == nullptr || counts1 == nullptr || src == nullptr ||
        (ns > 0 && ns_rows1 == nullptr))
        return TB200_ERR_NULL;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    pyramid_kept_rows_kernel<<<static_cast<unsigned>(batch), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        cu0, cu1, counts0, counts1, ns, src, ns_rows1, row_dst);
    count_launch();
    return launch_status();
}

extern "C" int tb200_sequence_prepare(const int64_t* values, const int64_t* lengths, const int64_t* timestamps,
                                      const int64_t* request_ts, int64_t batch, int32_t n_feat, int32_t max_len,
                                      int64_t* out_len, int32_t* out_src, float* out_stats, void* stream) {
    using namespace tb200;
    if (batch < 0 || n_feat < 1 || max_len < 1 || max_len > 8192) return TB200_ERR_SHAPE;
    if (batch == 0) return TB200_OK;
    if (values == nullptr || lengths == nullptr || timestamps == nullptr || request_ts == nullptr || out_len == nullptr ||
        out_src == nullptr || out_stats == nullptr)
        return TB200_ERR_NULL;
    if (batch > 0x7FFFFFFFll) return TB200_ERR_SHAPE;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    int table = 64;
    while (table < 2 * max_len) table <<= 1;
    const size_t smem = (static_cast<size_t>(2) * table + max_len + kThreads) * sizeof(int32_t);
    static bool attr_set[64] = {};
    const DeviceInfo& dev = device_info();
    if (!attr_set[dev.index]) {
        cudaFuncSetAttribute(seqprep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr_set[dev.index] = true;
    }
    seqprep_kernel<<<static_cast<unsigned>(batch), kThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        values, lengths, timestamps, request_ts, n_feat, max_len, table, out_len, out_src, out_stats);
    count_launch();
    return launch_status();
}

extern "C" int tb200_packed_token_index(const int64_t* values, const int64_t* timestamps, const int64_t* request_ts,
                                        const int32_t* src, const int64_t* cu_rows, const int64_t* seq_count,
                                        const int64_t* start, const int64_t* edges, int32_t n_edges,
                                        const int64_t* hash_buckets, int64_t batch, int32_t n_feat, int32_t max_len,
                                        int64_t total_rows, int64_t* ids_out, int64_t* pos_out, int64_t* bucket_out,
                                        void* stream) {
    using namespace tb200;
    if (batch < 0 || n_feat < 1 || max_len < 1 || total_rows < 0 || n_edges < 0) return TB200_ERR_SHAPE;
    if (batch == 0 || total_rows == 0) return TB200_OK;
    if (values == nullptr || request_ts == nullptr || src == nullptr || cu_rows == nullptr || seq_count == nullptr ||
        start == nullptr || hash_buckets == nullptr || ids_out == nullptr || pos_out == nullptr)
        return TB200_ERR_NULL;
    if (bucket_out != nullptr && (timestamps == nullptr || edges == nullptr || n_edges < 1)) return TB200_ERR_NULL;
    if (batch > 0x7FFFFFFFll) return TB200_ERR_SHAPE;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    token_index_kernel<<<static_cast<unsigned>(batch), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        values, timestamps, request_ts, src, cu_rows, seq_count, start, edges, n_edges, hash_buckets, n_feat, max_len,
        total_rows, ids_out, pos_out, bucket_out);
    count_launch();
    return launch_status();
}
