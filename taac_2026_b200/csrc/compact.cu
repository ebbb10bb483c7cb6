// Compact host format of the behaviour sequences and its expansion on the device.
//
// The reference's batch converter hands the model padded int64 buffers: ids [B, F, L], timestamps [B, L], lengths [B]
// (`PCVRRecordBatchConverter._build_sequence_inputs`, src/taac2026/infrastructure/data/batch_converter.py:446-488),
// and the evaluation loop copies them to the device as they are (application/evaluation/workflow.py:246-262).  At
// B 8192, L 1024 that is 134 MB per batch, more than half of it padding, all of it 64-bit.  The compact format keeps
// only the valid prefix of every sample, 32 bits per value:
//     cu[B + 1]        int32   cu[b] = first event of sample b, cu[B] = total number of events
//     ids[F, stride]   int32   ids[f, cu[b] + l] = values[b, f, l]                         (l < lengths[b])
//     gaps[total]      int32   request_timestamp[b] - timestamps[b, l], or kNoTimestamp where the timestamp is 0
// The host packers below write it (from the padded buffers, or straight from Arrow list columns — offsets + values —
// with the rule of `pad_list_offsets_values`, batch_converter.py:68-103, and of `_fill_sequence`, :503-538); the
// device kernel `expand_sequence_kernel` rebuilds the padded int64 tensors bit for bit in HBM, where writing 200 MB
// costs some 40 us instead of 20 ms on the PCIe link.  A value that does not fit 32 bits makes the packer refuse the
// batch (TB200_ERR_RANGE) so that the caller can fall back to the padded copy: nothing is ever truncated.
#include <algorithm>
#include <atomic>
#include <climits>
#include <cstring>
#include <thread>
#include <vector>

#include "tb200_common.cuh"

namespace tb200 {
void count_launch();

namespace {

constexpr int32_t kNoTimestamp = INT32_MIN;     // gap code of a zero (missing) timestamp

template <typename Fn>
void parallel_rows(int64_t rows, int threads, Fn fn) {
    int n = threads < 1 ? 1 : (threads > 64 ? 64 : threads);
    if (rows < 256 * static_cast<int64_t>(n)) n = static_cast<int>(std::max<int64_t>(1, rows / 256));
    if (n <= 1) {
        fn(0, rows);
        return;
    }
    std::vector<std::thread> pool;
    pool.reserve(n);
    const int64_t step = (rows + n - 1) / n;
    for (int t = 0; t < n; ++t) {
        const int64_t lo = t * step, hi = std::min(rows, lo + step);
        if (lo >= hi) break;
        pool.emplace_back([=] { fn(lo, hi); });
    }
    for (auto& th : pool) th.join();
}

inline bool fits32(int64_t v) { return v > INT32_MIN && v <= INT32_MAX; }   // INT32_MIN itself is the "no timestamp" code

inline int64_t offset_at(const void* offsets, int wide, int64_t i) {
    return wide ? static_cast<const int64_t*>(offsets)[i] : static_cast<int64_t>(static_cast<const int32_t*>(offsets)[i]);
}

// One thread per (sample, group of 2 positions): 16-byte stores of int64 pairs; positions at or beyond the
// sample's length get zeros, so the outputs need no memset.
__global__ void __launch_bounds__(256)
expand_sequence_kernel(const int32_t* __restrict__ ids, const int32_t* __restrict__ gaps, const int32_t* __restrict__ cu,
                       const int64_t* __restrict__ request_ts, int64_t* __restrict__ values, int64_t* __restrict__ lengths,
                       int64_t* __restrict__ timestamps, int batch, int feats, int max_len, int64_t ids_stride) {
    const int pairs = max_len >> 1;                      // max_len is even
    const int64_t total = static_cast<int64_t>(batch) * pairs;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total;
         i += static_cast<int64_t>(gridDim.x) * blockDim.x) {
        const int b = static_cast<int>(i / pairs);
        const int l = static_cast<int>(i - static_cast<int64_t>(b) * pairs) * 2;
        const int32_t first = cu[b];
        const int len = min(max(cu[b + 1] - first, 0), max_len);
        if (l == 0) lengths[b] = len;
        const bool in0 = l < len, in1 = l + 1 < len;
        const int64_t src = static_cast<int64_t>(first) + l;
        for (int f = 0; f < feats; ++f) {
            longlong2 v;
            v.x = in0 ? static_cast<int64_t>(ids[f * ids_stride + src]) : 0;
            v.y = in1 ? static_cast<int64_t>(ids[f * ids_stride + src + 1]) : 0;
            *reinterpret_cast<longlong2*>(values + (static_cast<int64_t>(b) * feats + f) * max_len + l) = v;
        }
        if (timestamps != nullptr) {
            const int64_t now = request_ts[b];
            longlong2 t = make_longlong2(0, 0);
            if (in0) { const int32_t g = gaps[src]; t.x = g == kNoTimestamp ? 0 : now - static_cast<int64_t>(g); }
            if (in1) { const int32_t g = gaps[src + 1]; t.y = g == kNoTimestamp ? 0 : now - static_cast<int64_t>(g); }
            *reinterpret_cast<longlong2*>(timestamps + static_cast<int64_t>(b) * max_len + l) = t;
        }
    }
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_expand_sequence(const int32_t* ids, const int32_t* gaps, const int32_t* cu, const int64_t* request_ts,
                                     int64_t* values, int64_t* lengths, int64_t* timestamps, int32_t batch, int32_t feats,
                                     int32_t max_len, int64_t ids_stride, void* stream) {
    using namespace tb200;
    if (batch < 0 || feats < 1 || max_len < 2 || ids_stride < 0) return TB200_ERR_SHAPE;
    if (max_len % 2 != 0) return TB200_ERR_ALIGN;
    if (batch == 0) return TB200_OK;
    if (ids == nullptr || cu == nullptr || values == nullptr || lengths == nullptr) return TB200_ERR_NULL;
    if (timestamps != nullptr && (gaps == nullptr || request_ts == nullptr)) return TB200_ERR_NULL;
    if (!aligned16(values) || (timestamps != nullptr && !aligned16(timestamps))) return TB200_ERR_ALIGN;
    const DeviceInfo& dev = device_info();
    if (!dev.valid) return TB200_ERR_DEVICE;
    const int64_t total = static_cast<int64_t>(batch) * (max_len / 2);
    int64_t grid = (total + 255) / 256;
    grid = std::min<int64_t>(grid, static_cast<int64_t>(dev.sm_count) * 16);
    expand_sequence_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        ids, gaps, cu, request_ts, values, lengths, timestamps, batch, feats, max_len, ids_stride);
    count_launch();
    return launch_status();
}

// ---- host side: no CUDA call below this line ----------------------------------------------------------------------

extern "C" int tb200_host_compact_offsets(const int64_t* lengths, int32_t batch, int32_t max_len, int32_t* cu) {
    if (batch < 0 || max_len < 0) return TB200_ERR_SHAPE;
    if (cu == nullptr || (batch > 0 && lengths == nullptr)) return TB200_ERR_NULL;
    int64_t total = 0;
    cu[0] = 0;
    for (int32_t b = 0; b < batch; ++b) {
        total += std::min<int64_t>(std::max<int64_t>(lengths[b], 0), max_len);
        if (total > INT32_MAX) return TB200_ERR_RANGE;
        cu[b + 1] = static_cast<int32_t>(total);
    }
    return TB200_OK;
}

extern "C" int tb200_host_compact_sequence(const int64_t* values, const int64_t* timestamps, const int64_t* request_ts,
                                           const int32_t* cu, int32_t batch, int32_t feats, int32_t max_len, int32_t* ids,
                                           int64_t ids_stride, int32_t* gaps, int32_t threads) {
    using namespace tb200;
    if (batch < 0 || feats < 1 || max_len < 0) return TB200_ERR_SHAPE;
    if (batch == 0) return TB200_OK;
    if (values == nullptr || cu == nullptr || ids == nullptr) return TB200_ERR_NULL;
    if (gaps != nullptr && (timestamps == nullptr || request_ts == nullptr)) return TB200_ERR_NULL;
    if (ids_stride < cu[batch]) return TB200_ERR_SHAPE;
    std::atomic<int> bad{0};
    parallel_rows(batch, threads, [&](int64_t lo, int64_t hi) {
        bool ok = true;
        for (int64_t b = lo; b < hi; ++b) {
            const int64_t first = cu[b];
            const int64_t len = cu[b + 1] - first;
            for (int f = 0; f < feats; ++f) {
                const int64_t* src = values + (b * feats + f) * max_len;
                int32_t* dst = ids + f * ids_stride + first;
                for (int64_t l = 0; l < len; ++l) {
                    ok &= src[l] >= INT32_MIN && src[l] <= INT32_MAX;
                    dst[l] = static_cast<int32_t>(src[l]);
                }
            }
            if (gaps != nullptr) {
                const int64_t* ts = timestamps + b * max_len;
                const int64_t now = request_ts[b];
                for (int64_t l = 0; l < len; ++l) {
                    const int64_t gap = now - ts[l];
                    const bool none = ts[l] == 0;
                    ok &= none || fits32(gap);
                    gaps[first + l] = none ? kNoTimestamp : static_cast<int32_t>(gap);
                }
            }
        }
        if (!ok) bad.store(1, std::memory_order_relaxed);
    });
    return bad.load() ? TB200_ERR_RANGE : TB200_OK;
}

// Arrow list columns in, compact format out.  Rule per column (pad_list_offsets_values): a row contributes its first
// min(end - start, max_len) values; the sample's length is the largest such count over the id columns (_fill_sequence),
// shorter columns are zero-filled up to it; ids <= 0 become 0 (_build_sequence_inputs: `tokens[tokens <= 0] = 0`); the
// timestamp column follows the same prefix rule and positions it does not cover count as "no timestamp".  With
// vocab_sizes given, the out-of-vocabulary rule of `_clip_sequence_vocab` / `record_oob` (:594-650) is applied as
// under clip_vocab=True: a column whose vocabulary size is <= 0 is all zeros, ids >= the size become 0 and are
// counted per column in oob_counts (a caller that does not clip raises when a count is not zero).
extern "C" int tb200_host_compact_from_lists(const void* const* id_offsets, const int64_t* const* id_values, int32_t feats,
                                             const void* ts_offsets, const int64_t* ts_values, int32_t offsets_are_int64,
                                             const int64_t* request_ts, const int64_t* vocab_sizes, int64_t* oob_counts,
                                             int32_t batch, int32_t max_len, int32_t* cu,
                                             int32_t* ids, int64_t ids_stride, int32_t* gaps, int32_t threads) {
    using namespace tb200;
    if (batch < 0 || feats < 1 || max_len < 0) return TB200_ERR_SHAPE;
    if (cu == nullptr || id_offsets == nullptr || id_values == nullptr) return TB200_ERR_NULL;
    for (int f = 0; f < feats; ++f)
        if (id_offsets[f] == nullptr || id_values[f] == nullptr) return TB200_ERR_NULL;
    if (gaps != nullptr && ts_offsets != nullptr && (ts_values == nullptr || request_ts == nullptr)) return TB200_ERR_NULL;
    int64_t total = 0;
    cu[0] = 0;
    for (int32_t b = 0; b < batch; ++b) {
        int64_t len = 0;
        for (int f = 0; f < feats; ++f) {
            const int64_t raw = offset_at(id_offsets[f], offsets_are_int64, b + 1) - offset_at(id_offsets[f], offsets_are_int64, b);
            len = std::max(len, std::min<int64_t>(std::max<int64_t>(raw, 0), max_len));
        }
        total += len;
        if (total > INT32_MAX) return TB200_ERR_RANGE;
        cu[b + 1] = static_cast<int32_t>(total);
    }
    if (oob_counts != nullptr) std::memset(oob_counts, 0, static_cast<size_t>(feats) * sizeof(int64_t));
    if (batch == 0 || total == 0) return TB200_OK;
    if (ids == nullptr) return TB200_ERR_NULL;
    if (ids_stride < total || feats > 256) return TB200_ERR_SHAPE;
    std::atomic<int> bad{0};
    std::vector<std::atomic<int64_t>> oob(feats);
    for (auto& c : oob) c.store(0);
    parallel_rows(batch, threads, [&](int64_t lo, int64_t hi) {
        bool ok = true;
        int64_t oob_local[256] = {};
        for (int64_t b = lo; b < hi; ++b) {
            const int64_t first = cu[b];
            const int64_t len = cu[b + 1] - first;
            for (int f = 0; f < feats; ++f) {
                const int64_t start = offset_at(id_offsets[f], offsets_are_int64, b);
                const int64_t raw = offset_at(id_offsets[f], offsets_are_int64, b + 1) - start;
                const int64_t use = std::min<int64_t>(std::max<int64_t>(raw, 0), len);
                const int64_t* src = id_values[f] + start;
                int32_t* dst = ids + f * ids_stride + first;
                const bool clip = vocab_sizes != nullptr;
                const int64_t vocab = clip ? vocab_sizes[f] : 0;
                for (int64_t l = 0; l < use; ++l) {
                    int64_t v = src[l] > 0 ? src[l] : 0;
                    if (clip && v >= vocab) {
                        oob_local[f] += vocab > 0 ? 1 : 0;
                        v = 0;
                    }
                    ok &= v <= INT32_MAX;
                    dst[l] = static_cast<int32_t>(v);
                }
                if (use < len) std::memset(dst + use, 0, static_cast<size_t>(len - use) * sizeof(int32_t));
            }
            if (gaps != nullptr) {
                int64_t use = 0, start = 0;
                if (ts_offsets != nullptr) {
                    start = offset_at(ts_offsets, offsets_are_int64, b);
                    const int64_t raw = offset_at(ts_offsets, offsets_are_int64, b + 1) - start;
                    use = std::min<int64_t>(std::max<int64_t>(raw, 0), len);
                }
                const int64_t now = request_ts != nullptr ? request_ts[b] : 0;
                for (int64_t l = 0; l < use; ++l) {
                    const int64_t t = ts_values[start + l];
                    const int64_t gap = now - t;
                    ok &= t == 0 || fits32(gap);
                    gaps[first + l] = t == 0 ? kNoTimestamp : static_cast<int32_t>(gap);
                }
                for (int64_t l = use; l < len; ++l) gaps[first + l] = kNoTimestamp;
            }
        }
        for (int f = 0; f < feats; ++f)
            if (oob_local[f] != 0) oob[f].fetch_add(oob_local[f], std::memory_order_relaxed);
        if (!ok) bad.store(1, std::memory_order_relaxed);
    });
    if (oob_counts != nullptr)
        for (int f = 0; f < feats; ++f) oob_counts[f] = oob[f].load();
    return bad.load() ? TB200_ERR_RANGE : TB200_OK;
}

// The converter's strict time filter (`_fill_strict_sequence` / `_copy_strict_side_columns`, batch_converter.py:540-592):
// a row keeps the positions p of its timestamp list with 0 < ts[p] < request_ts, the last max_len of them; its
// length is their number and its timestamps are theirs.  An id column contributes values[start + p] for the kept
// positions below its own length, written from slot 0 on (so a short id column is compacted to the front, as the
// reference does), zeros behind; ids <= 0 -> 0 and the vocabulary rule as above.
extern "C" int tb200_host_compact_from_lists_strict(const void* const* id_offsets, const int64_t* const* id_values, int32_t feats,
                                                    const void* ts_offsets, const int64_t* ts_values, int32_t offsets_are_int64,
                                                    const int64_t* request_ts, const int64_t* vocab_sizes, int64_t* oob_counts,
                                                    int32_t batch, int32_t max_len, int32_t* cu, int32_t* ids,
                                                    int64_t ids_stride, int32_t* gaps, int32_t threads) {
    using namespace tb200;
    if (batch < 0 || feats < 1 || max_len < 0 || feats > 256) return TB200_ERR_SHAPE;
    if (cu == nullptr || id_offsets == nullptr || id_values == nullptr || ts_offsets == nullptr || ts_values == nullptr ||
        request_ts == nullptr)
        return TB200_ERR_NULL;
    for (int f = 0; f < feats; ++f)
        if (id_offsets[f] == nullptr || id_values[f] == nullptr) return TB200_ERR_NULL;
    auto is_valid = [](int64_t t, int64_t now) { return t > 0 && t < now; };
    // phase 1: lengths (in parallel, parked in cu[b + 1]), then the prefix sum
    parallel_rows(batch, threads, [&](int64_t lo, int64_t hi) {
        for (int64_t b = lo; b < hi; ++b) {
            const int64_t start = offset_at(ts_offsets, offsets_are_int64, b);
            const int64_t end = offset_at(ts_offsets, offsets_are_int64, b + 1);
            int64_t n = 0;
            for (int64_t p = start; p < end; ++p) n += is_valid(ts_values[p], request_ts[b]) ? 1 : 0;
            cu[b + 1] = static_cast<int32_t>(std::min<int64_t>(n, max_len));
        }
    });
    int64_t total = 0;
    cu[0] = 0;
    for (int32_t b = 0; b < batch; ++b) {
        total += cu[b + 1];
        if (total > INT32_MAX) return TB200_ERR_RANGE;
        cu[b + 1] = static_cast<int32_t>(total);
    }
    if (oob_counts != nullptr) std::memset(oob_counts, 0, static_cast<size_t>(feats) * sizeof(int64_t));
    if (batch == 0 || total == 0) return TB200_OK;
    if (ids == nullptr) return TB200_ERR_NULL;
    if (ids_stride < total) return TB200_ERR_SHAPE;
    std::atomic<int> bad{0};
    std::vector<std::atomic<int64_t>> oob(feats);
    for (auto& c : oob) c.store(0);
    parallel_rows(batch, threads, [&](int64_t lo, int64_t hi) {
        bool ok = true;
        int64_t oob_local[256] = {};
        std::vector<int64_t> kept;           // kept positions of the row, relative to the start of its lists
        for (int64_t b = lo; b < hi; ++b) {
            const int64_t first = cu[b];
            const int64_t len = cu[b + 1] - first;
            if (len == 0) continue;
            const int64_t start = offset_at(ts_offsets, offsets_are_int64, b);
            const int64_t end = offset_at(ts_offsets, offsets_are_int64, b + 1);
            const int64_t now = request_ts[b];
            kept.clear();
            for (int64_t p = start; p < end; ++p)
                if (is_valid(ts_values[p], now)) kept.push_back(p - start);
            const int64_t skip = static_cast<int64_t>(kept.size()) - len;      // only the last `len` positions stay
            for (int64_t j = 0; j < len; ++j) {
                const int64_t gap = now - ts_values[start + kept[skip + j]];
                ok &= fits32(gap);
                if (gaps != nullptr) gaps[first + j] = static_cast<int32_t>(gap);
            }
            for (int f = 0; f < feats; ++f) {
                const int64_t f_start = offset_at(id_offsets[f], offsets_are_int64, b);
                const int64_t side_len = offset_at(id_offsets[f], offsets_are_int64, b + 1) - f_start;
                int32_t* dst = ids + f * ids_stride + first;
                const bool clip = vocab_sizes != nullptr;
                const int64_t vocab = clip ? vocab_sizes[f] : 0;
                int64_t n = 0;
                for (int64_t j = 0; j < len; ++j) {
                    const int64_t p = kept[skip + j];
                    if (p >= side_len) break;                                   // positions are increasing
                    int64_t v = id_values[f][f_start + p];
                    v = v > 0 ? v : 0;
                    if (clip && v >= vocab) {
                        oob_local[f] += vocab > 0 ? 1 : 0;
                        v = 0;
                    }
                    ok &= v <= INT32_MAX;
                    dst[n++] = static_cast<int32_t>(v);
                }
                if (n < len) std::memset(dst + n, 0, static_cast<size_t>(len - n) * sizeof(int32_t));
            }
        }
        for (int f = 0; f < feats; ++f)
            if (oob_local[f] != 0) oob[f].fetch_add(oob_local[f], std::memory_order_relaxed);
        if (!ok) bad.store(1, std::memory_order_relaxed);
    });
    if (oob_counts != nullptr)
        for (int f = 0; f < feats; ++f) oob_counts[f] = oob[f].load();
    return bad.load() ? TB200_ERR_RANGE : TB200_OK;
}
