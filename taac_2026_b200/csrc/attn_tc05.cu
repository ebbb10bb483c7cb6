// Varlen masked attention forward on the 5th-generation tensor cores (sm_100a): head_dim 64, bf16.
//
// Persistent CTAs walk the work items (128 query rows of one sample and head); two CTAs fit an SM
// (256 TMEM columns and 97 KB of shared memory each), so one runs its softmax while the other owns the
// tensor cores, and the TMA producer of a CTA already fetches the next item's Q / K / V while the
// current item is being finished.  Roles (192 threads):
//   warp 0       TMA producer: Q per item, K and V tiles alternating through one ring of five slots
//                (128 keys x 128 bytes each, 128-byte swizzle, no multicast)
//   warp 1       MMA issuer (one elected lane), owner of the TMEM allocation
//   warps 2..5   softmax: one thread per query row
// TMEM columns of a CTA: S 0..127 (fp32 scores), O 128..191 (fp32 output), P 192..255 (bf16 probabilities, two per
// column).  Per KV tile:  S = Q K^T   (tcgen05.mma kind::f16, both operands from shared memory, M 128 x N 128 x K 64)
//                        the softmax thread reads its S row with x16 tcgen05.ld pairs (32 columns per wait group),
//                        takes the row maximum, frees S as soon as the row has been read, and writes
//                        P = exp2(...) as bf16 straight back into TMEM (tcgen05.st): no shared-memory round trip
//                        O += P V    (P is the TMEM operand, V the MN-major shared-memory operand, M 128 x N 64 x
//                        K 128, issued in two halves so that the first runs while the softmax finishes the
//                        second), accumulated in TMEM across the key tiles.  The running max is only advanced
//                        when it grows by more than 2^8 (the exponent stays within fp32 / bf16 range, the final
//                        division by the row sum makes the result exact); when it does, the threads
//                        rescale their O rows in TMEM (tcgen05.ld / tcgen05.st) before P is released.
// Key tiles without a visible key are skipped; masks come as lengths, never as a matrix.
// Every mbarrier wait is bounded; a wait that gives up raises the status word and all roles drain
// through the final barrier, where TMEM is released.
#include <cudaTypedefs.h>

#include <type_traits>

#include "attn_common.cuh"
#include "tb200_common.cuh"
#include "tb200_ptx.cuh"

namespace tb200 {
void count_launch();

namespace {

constexpr int kD = 64;            // head dim
constexpr int kHalf = 128;        // query rows per half == TMEM lanes
constexpr int kHalves = 1;        // 128-row query blocks per CTA (two CTAs share an SM and overlap each other)
constexpr int kBM = kHalves * kHalf;  // query rows per CTA
constexpr int kBN = 128;          // keys per tile
constexpr int kThreads = 64 + kHalves * 128;
constexpr int kSoftmaxThreads = 128;  // per half
constexpr uint32_t kTileBytes = kBN * kD * 2;       // 16 KB: one Q half, K tile or V tile
constexpr uint32_t kSlots = 5;                      // K / V tile ring
constexpr uint32_t kTmemCols = kHalves == 1 ? 256 : 512;
// TMEM columns: S of half h at h * 128, O of half h behind the S blocks at h * 64
constexpr uint32_t kTmemS = 0;
constexpr uint32_t kTmemO = kHalves * 128;
// P (bf16 probabilities, two per 32-bit column) is the TMEM A operand of the P V product
constexpr uint32_t kTmemP = kTmemO + kHalves * 64;

struct Tc05Args {
    AttnArgs a;
    int32_t* status;
};

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Per-CTA description of which key tiles each half works on; every role derives the same sequence.
struct Plan {
    int lq, lk, valid_len, ns_start, m0;
    bool causal, self_rows, packed;
    int64_t row_base;     // packed: first row of the sample
    int n_tiles;          // key tiles that any half may need
    int kv_end[2];        // keys [0, kv_end[h]) can be visible to half h
    bool half_on[2];      // half has rows to compute
    __device__ __forceinline__ bool live(int j) const {
        const int n0 = j * kBN;
        return n0 < valid_len || n0 + kBN > ns_start;
    }
    __device__ __forceinline__ bool active(int j, int h) const { return half_on[h] && live(j) && j * kBN < kv_end[h]; }
};

__device__ __forceinline__ Plan make_plan(const AttnArgs& a, int b, int m0) {
    Plan p;
    p.packed = a.cu_rows != nullptr;
    p.lq = a.Lq;
    p.lk = a.Lk;
    p.row_base = 0;
    if (p.packed) {
        p.row_base = a.cu_rows[b];
        p.lq = p.lk = a.cu_rows[b + 1] - static_cast<int32_t>(p.row_base);
    }
    p.m0 = m0;
    p.valid_len = (a.seq_len != nullptr && !p.packed) ? min(max(a.seq_len[b], 0), p.lk) : p.lk;
    p.ns_start = p.packed ? p.lk : min(a.ns_start, p.lk);
    p.causal = a.causal != 0;
    p.self_rows = a.padded_query_self != 0;
    int n_max = 0;
    p.half_on[1] = false;
    p.kv_end[1] = 0;
    for (int h = 0; h < kHalves; ++h) {
        const int r0 = m0 + h * kHalf;
        const int r1 = min(r0 + kHalf, p.lq);
        // a half wholly inside the padded query range only copies value rows
        const bool all_padded = p.self_rows && r0 >= p.valid_len && r1 <= p.ns_start;
        p.half_on[h] = r0 < p.lq && !all_padded;
        p.kv_end[h] = p.causal ? min(p.lk, r1) : p.lk;
        if (p.half_on[h]) n_max = max(n_max, (p.kv_end[h] + kBN - 1) / kBN);
    }
    p.n_tiles = n_max;
    return p;
}

__device__ __forceinline__ float max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// Work items: (query block of 128 rows, head, sample), walked in the same order by every role of a
// persistent CTA (item w = blockIdx.x + i * gridDim.x).  Two orders of the item list:
//   block-major (rows of equal length): later query blocks come first; under a causal mask they own the most key
//     tiles, so the long items start early and the short ones fill the tail;
//   sample-major (ragged batches: a length vector or packed rows): all blocks and heads of a sample are neighbours in
//     the list, so the CTAs that run at the same time read the K / V tiles of a few samples and find them in the L2
//     (measured on 256 samples of 32..1024 keys: 4-5 % faster, causal or not; on equal lengths under a causal mask
//     the block-major order is the faster one by the same margin).
struct Work {
    int n_qb, heads, batch;
    int64_t total;
    bool sample_major;
    __device__ __forceinline__ void decode(int64_t w, int& qb, int& h, int& b) const {
        if (sample_major) {
            const int per_b = n_qb * heads;
            b = static_cast<int>(w / per_b);
            const int rem = static_cast<int>(w % per_b);
            qb = n_qb - 1 - rem / heads;
            h = rem % heads;
            return;
        }
        const int64_t per_qb = static_cast<int64_t>(heads) * batch;
        qb = n_qb - 1 - static_cast<int>(w / per_qb);
        const int rem = static_cast<int>(w % per_qb);
        h = rem % heads;
        b = rem / heads;
    }
};

__global__ void __launch_bounds__(kThreads, 2)
attn_tc05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_k,
                 const __grid_constant__ CUtensorMap tmap_v, const Tc05Args args) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t q_full, q_empty;
    __shared__ uint64_t kv_full[kSlots], kv_empty[kSlots];  // one ring of tile slots: K_0, V_0, K_1, V_1, ...
    __shared__ uint64_t s_full, s_free, p_full[2], o_full;   // p_full[i]: P of keys [64 i, 64 i + 64) of the tile is in TMEM
    __shared__ uint32_t tmem_base_slot;

    const AttnArgs& a = args.a;
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* sQ = smem;                              // 16 KB
    uint8_t* sKV = sQ + kTileBytes;                  // kSlots x 16 KB: K and V tiles alternate through one ring,
                                                     // so the tiles of the next two steps are in flight during tile j

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    Work work;
    work.n_qb = (a.Lq + kBM - 1) / kBM;
    work.heads = a.H;
    work.batch = a.B;
    work.total = static_cast<int64_t>(work.n_qb) * a.H * a.B;
    work.sample_major = a.seq_len != nullptr || a.cu_rows != nullptr;

    if (threadIdx.x == 0) {
        mbar_init(&q_full, 1);
        mbar_init(&q_empty, 1);
        for (int i = 0; i < static_cast<int>(kSlots); ++i) {
            mbar_init(&kv_full[i], 1);
            mbar_init(&kv_empty[i], 1);
        }
        mbar_init(&s_full, 1);
        mbar_init(&s_free, kSoftmaxThreads);
        mbar_init(&p_full[0], kSoftmaxThreads);
        mbar_init(&p_full[1], kSoftmaxThreads);
        mbar_init(&o_full, 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_slot, kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tmap_q);
            tma_prefetch_desc(&tmap_k);
            tma_prefetch_desc(&tmap_v);
            uint32_t qc = 0, kc = 0;
            bool ok = true;
            for (int64_t w = blockIdx.x; w < work.total && ok; w += gridDim.x) {
                int qb, h_idx, b;
                work.decode(w, qb, h_idx, b);
                const Plan plan = make_plan(a, b, qb * kBM);
                if (!plan.half_on[0] || plan.n_tiles == 0) continue;
                // TMA coordinates: (d, row, head, batch); packed batches address rows of the whole matrix
                const int row0 = plan.packed ? static_cast<int>(plan.row_base) : 0;
                const int bz = plan.packed ? 0 : b;
                if (!mbar_wait_sleep(&q_empty, (qc & 1) ^ 1)) { ok = false; break; }
                mbar_expect_tx(&q_full, kTileBytes);
                tma_load_4d(sQ, &tmap_q, 0, row0 + plan.m0, h_idx, bz, &q_full);
                ++qc;
                for (int j = 0; j < plan.n_tiles && ok; ++j) {
                    if (!plan.active(j, 0)) continue;
                    for (int which = 0; which < 2; ++which) {  // K tile, then V tile
                        const uint32_t t = 2 * kc + which;
                        const uint32_t slot = t % kSlots;
                        if (!mbar_wait_sleep(&kv_empty[slot], ((t / kSlots) & 1) ^ 1)) { ok = false; break; }
                        mbar_expect_tx(&kv_full[slot], kTileBytes);
                        tma_load_4d(sKV + slot * kTileBytes, which == 0 ? &tmap_k : &tmap_v, 0, row0 + j * kBN, h_idx, bz,
                                    &kv_full[slot]);
                    }
                    ++kc;
                }
            }
            if (!ok) {
                if (args.status != nullptr) atomicExch(args.status, 1);
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (lane == 0) {
            const uint32_t idesc_s = umma_idesc(1, 1, 0, 0, kHalf, kBN);  // bf16 x bf16, Q and K both K-major
            const uint32_t idesc_o = umma_idesc(1, 1, 0, 1, kHalf, kD);   // P K-major, V MN-major (head dim contiguous)
            const uint32_t q_addr = smem_u32(sQ);
            uint32_t qc = 0, kc = 0;
            bool ok = true;
            for (int64_t w = blockIdx.x; w < work.total && ok; w += gridDim.x) {
                int qb, h_idx, b;
                work.decode(w, qb, h_idx, b);
                const Plan plan = make_plan(a, b, qb * kBM);
                if (!plan.half_on[0] || plan.n_tiles == 0) continue;
                if (!mbar_wait_sleep(&q_full, qc & 1)) { ok = false; break; }
                ++qc;
                // S of tile j + 1 is issued before P V of tile j: the softmax of j runs from registers, so the
                // tensor cores fill the S buffer again while it computes
                auto issue_s = [&](uint32_t tile_index, bool last_of_item) -> bool {
                    const uint32_t t = 2 * tile_index;
                    const uint32_t slot = t % kSlots;
                    if (!mbar_wait_sleep(&kv_full[slot], (t / kSlots) & 1) || !mbar_wait_sleep(&s_free, (tile_index & 1) ^ 1)) return false;
                    tc_fence_after_sync();
                    const uint32_t k_addr = smem_u32(sKV + slot * kTileBytes);
#pragma unroll
                    for (int k = 0; k < kD / 16; ++k) {
                        mma_f16_ss(tmem_base + kTmemS, umma_desc_sw128(q_addr + k * 32, 1024, 16),
                                   umma_desc_sw128(k_addr + k * 32, 1024, 16), idesc_s, k > 0 ? 1u : 0u);
                    }
                    tc_commit(&s_full);
                    tc_commit(&kv_empty[slot]);             // K tile free once the S product has read it
                    if (last_of_item) tc_commit(&q_empty);   // and so is Q after the item's last S product
                    return true;
                };
                int n_active = 0;
                for (int j = 0; j < plan.n_tiles; ++j) n_active += plan.active(j, 0) ? 1 : 0;
                if (n_active == 0) {          // nothing visible: hand Q back to the producer directly
                    mbar_arrive(&q_empty);
                    continue;
                }
                // Per tile the issuer follows the order in which the softmax warps release things: first half of P
                // -> P V over keys [0, 64); S buffer free -> S of the next tile; second half of P -> rest of P V.
                // The first half of P V and the next S product run while the softmax still works on the tile.
                if (!issue_s(kc, n_active == 1)) { ok = false; break; }
                for (int i = 0; i < n_active && ok; ++i) {
                    const uint32_t t = 2 * kc + 1;
                    const uint32_t slot = t % kSlots;
                    const uint32_t v_addr = smem_u32(sKV + slot * kTileBytes);
                    if (!mbar_wait_sleep(&kv_full[slot], (t / kSlots) & 1)) { ok = false; break; }
#pragma unroll 1
                    for (int half = 0; half < 2; ++half) {
                        if (half == 1 && i + 1 < n_active && !issue_s(kc + 1, i + 2 == n_active)) { ok = false; break; }
                        if (!mbar_wait_sleep(&p_full[half], kc & 1)) { ok = false; break; }
                        tc_fence_after_sync();
#pragma unroll
                        for (int kk = 0; kk < kBN / 32; ++kk) {
                            const int k = half * (kBN / 32) + kk;
                            // A: P from TMEM, 16 keys = 8 columns per step; B: V, MN-major, 16 key rows = 2 KB per step
                            mma_f16_ts(tmem_base + kTmemO, tmem_base + kTmemP + k * 8,
                                       umma_desc_sw128(v_addr + k * 2048, 1024, 1024), idesc_o, (k > 0 || i > 0) ? 1u : 0u);
                        }
                    }
                    if (!ok) break;
                    tc_commit(&o_full);
                    tc_commit(&kv_empty[slot]);
                    ++kc;
                }
            }
            if (!ok) {
                if (args.status != nullptr) atomicExch(args.status, 1);
            }
        }
    } else {
        // ------------------------------------------------------------------ softmax + output
        const int quarter = warp & 3;                  // TMEM lanes [32 * quarter, +32)
        const int r_local = quarter * 32 + lane;       // row inside the block
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        const uint32_t t_s = tmem_base + kTmemS + lane_addr;
        const uint32_t t_o = tmem_base + kTmemO + lane_addr;
        const uint32_t t_p = tmem_base + kTmemP + lane_addr;
        const float sl2 = a.scale_log2;
        uint32_t kc = 0;
        bool ok = true;

        for (int64_t w = blockIdx.x; w < work.total && ok; w += gridDim.x) {
            int qb, h_idx, b;
            work.decode(w, qb, h_idx, b);
            const int m0 = qb * kBM;
            const Plan plan = make_plan(a, b, m0);
            if (m0 >= plan.lq) continue;
            const int row = m0 + r_local;              // query index inside the sample
            // Visibility of key column c for this thread's row, as two half-open ranges:
            //   [0, lim_lo) and [ns_lo, lim_hi)  with lim_hi = min(lk, causal ? row + 1 : lk)
            const int lim_hi = plan.causal ? min(plan.lk, row + 1) : plan.lk;
            const int lim_lo = min(plan.valid_len, lim_hi);
            const int ns_lo = plan.ns_start;
            float m_ref = -INFINITY;   // reference max of the exponent (lags the true max by at most 2^8)
            float l_run = 0.f;
            int tiles_done = 0;

            // One KV tile.  FULL tiles (every key visible to every row) carry no mask code.  The tile is read from
            // TMEM twice (row max, then probabilities) in rolled loops over 32-column chunks: the instruction
            // footprint stays small enough for the instruction caches, which a fully unrolled 128-column body
            // held in registers did not.
            auto tile = [&](const int n0, auto full_tag) -> bool {
                constexpr bool FULL = decltype(full_tag)::value;
                if (!mbar_wait_sleep(&s_full, kc & 1)) return false;
                tc_fence_after_sync();
                // visibility of the 32 columns from `base` on as a bit mask
                auto chunk_mask = [&](const int base) -> uint32_t {
                    auto low = [](int k) -> uint32_t { return k <= 0 ? 0u : (k >= 32 ? 0xffffffffu : ((1u << k) - 1u)); };
                    return low(lim_lo - base) | (low(lim_hi - base) & ~low(ns_lo - base));
                };

                // pass 1, row max: the four chunk loads are issued together, so one TMEM latency is exposed
                float mx0 = -INFINITY, mx1 = -INFINITY;
                uint32_t chunk_live = 0xfu;   // bit c: some row of the warp sees a key of chunk c
                {
                    uint32_t sr[4][32];
#pragma unroll
                    for (int c = 0; c < 4; ++c) tmem_ld_2x16(t_s + c * 32, sr[c]);
#pragma unroll
                    for (int c = 0; c < 4; ++c) tc_wait_ld(sr[c]);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        if (!FULL) {
                            const uint32_t vis = chunk_mask(n0 + c * 32);
                            // a chunk that no row of the warp can see (above the diagonal, past the keys) is
                            // skipped in both passes
                            if (!__any_sync(0xffffffffu, vis != 0u)) {
                                chunk_live &= ~(1u << c);
                                continue;
                            }
#pragma unroll
                            for (int i = 0; i < 32; ++i)
                                if (!((vis >> i) & 1u)) sr[c][i] = 0xff800000u;  // -inf
                        }
#pragma unroll
                        for (int i = 0; i < 32; i += 4) {
                            mx0 = max3(mx0, __uint_as_float(sr[c][i]), __uint_as_float(sr[c][i + 1]));
                            mx1 = max3(mx1, __uint_as_float(sr[c][i + 2]), __uint_as_float(sr[c][i + 3]));
                        }
                    }
                }
                const float mx = fmaxf(mx0, mx1);
                // advance the reference max only for a large jump (or on the first visible key of the row)
                float corr = 1.0f;
                bool grow = false;
                if (mx > m_ref && (m_ref == -INFINITY || (mx - m_ref) * sl2 > 8.0f)) {
                    corr = m_ref == -INFINITY ? 0.f : ex2((m_ref - mx) * sl2);
                    m_ref = mx;
                    grow = true;
                }
                const float ms = (m_ref == -INFINITY ? 0.f : m_ref) * sl2;

                // the previous P V of this item must be done before P is overwritten or O is rescaled
                if (tiles_done > 0) {
                    if (!mbar_wait_sleep(&o_full, (kc - 1) & 1)) return false;
                    tc_fence_after_sync();
                    if (__any_sync(0xffffffffu, grow)) {  // tcgen05.ld / st are warp-wide: corr = 1 where unchanged
                        const float2 corr2 = make_float2(corr, corr);
#pragma unroll 1
                        for (int c = 0; c < 2; ++c) {
                            uint32_t r[32];
                            tmem_ld_x32(t_o + c * 32, r);
                            tc_wait_ld();
#pragma unroll
                            for (int i = 0; i < 16; ++i) {
                                const float2 v = __fmul2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), corr2);
                                r[2 * i] = __float_as_uint(v.x);
                                r[2 * i + 1] = __float_as_uint(v.y);
                            }
                            tmem_st_x32(t_o + c * 32, r);
                        }
                        tc_wait_st();
                        tc_fence_before_sync();
                    }
                }

                // probabilities -> bf16 -> shared memory (K-major, 128-byte swizzle): chunk c covers keys
                // [32 c, 32 c + 32) = 4 x 16 bytes of the 64-key atom c / 2
                float2 sum2 = make_float2(0.f, 0.f);
                const float2 sl22 = make_float2(sl2, sl2);
                const float2 nms2 = make_float2(-ms, -ms);
                auto emit = [&](const int c, uint32_t (&r)[32]) {
                    if (!FULL) {
                        if (!((chunk_live >> c) & 1u)) {   // nothing visible to this warp: P = 0
                            uint32_t zero[16];
#pragma unroll
                            for (int i = 0; i < 16; ++i) zero[i] = 0u;
                            tmem_st_x16(t_p + c * 16, zero);
                            return;
                        }
                        const uint32_t vis = chunk_mask(n0 + c * 32);
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (!((vis >> i) & 1u)) r[i] = 0xff800000u;
                    }
                    uint32_t pk[16];
#pragma unroll
                    for (int i = 0; i < 16; ++i) {
                        const float2 sv = make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                        const float2 e = __ffma2_rn(sv, sl22, nms2);
                        const float2 p = make_float2(ex2(e.x), ex2(e.y));
                        sum2 = __fadd2_rn(sum2, p);
                        __nv_bfloat162 pb = __float22bfloat162_rn(p);
                        pk[i] = *reinterpret_cast<uint32_t*>(&pb);
                    }
                    tmem_st_x16(t_p + c * 16, pk);
                };
                // pass 2: the load of chunk c + 1 is in flight while chunk c is turned into probabilities
                {
                    uint32_t ra[32], rb[32];
                    tmem_ld_2x16(t_s, ra);
                    tc_wait_ld(ra);
#pragma unroll 1
                    for (int c = 0; c < 4; c += 2) {
                        tmem_ld_2x16(t_s + (c + 1) * 32, rb);
                        emit(c, ra);
                        tc_wait_ld(rb);
                        if (c == 0) {
                            tmem_ld_2x16(t_s + 2 * 32, ra);
                        } else {               // the whole row has been read: S may be overwritten
                            tc_fence_before_sync();
                            mbar_arrive(&s_free);
                        }
                        emit(c + 1, rb);
                        tc_wait_st();          // this half of P is in TMEM before the issuer is told
                        tc_fence_before_sync();
                        mbar_arrive(&p_full[c >> 1]);
                        if (c == 0) tc_wait_ld(ra);
                    }
                }
                l_run = l_run * corr + (sum2.x + sum2.y);
                ++kc;
                ++tiles_done;
                return true;
            };

            if (plan.half_on[0]) {
                for (int j = 0; j < plan.n_tiles && ok; ++j) {
                    if (!plan.active(j, 0)) continue;
                    const int n0 = j * kBN;
                    const bool full = (n0 + kBN <= plan.valid_len || n0 >= plan.ns_start) && n0 + kBN <= plan.lk &&
                                      (!plan.causal || n0 + kBN - 1 <= m0);
                    ok = full ? tile(n0, std::true_type{}) : tile(n0, std::false_type{});
                }
            }
            if (!ok) break;

            float2 o_acc[kD / 2];
#pragma unroll
            for (int i = 0; i < kD / 2; ++i) o_acc[i] = make_float2(0.f, 0.f);
            if (tiles_done > 0) {
                if (!mbar_wait_sleep(&o_full, (kc - 1) & 1)) { ok = false; break; }
                tc_fence_after_sync();
#pragma unroll
                for (int c = 0; c < 2; ++c) {
                    uint32_t r[32];
                    tmem_ld_x32(t_o + c * 32, r);
                    tc_wait_ld();
#pragma unroll
                    for (int i = 0; i < 16; ++i)
                        o_acc[c * 16 + i] = make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
                }
                tc_fence_before_sync();
            }
            if (row < plan.lq) {
                const int64_t o_off = (plan.packed ? plan.row_base * a.o_sl : static_cast<int64_t>(b) * a.o_sb) +
                                      static_cast<int64_t>(h_idx) * a.o_sh + static_cast<int64_t>(row) * a.o_sl;
                uint4* dst = reinterpret_cast<uint4*>(static_cast<__nv_bfloat16*>(a.o) + o_off);
                const bool padded_q = plan.self_rows && row >= plan.valid_len && row < plan.ns_start;
                if (padded_q) {
                    const int64_t v_off = (plan.packed ? plan.row_base * a.v_sl : static_cast<int64_t>(b) * a.v_sb) +
                                          static_cast<int64_t>(h_idx) * a.v_sh + static_cast<int64_t>(row) * a.v_sl;
                    const uint4* src = reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(a.v) + v_off);
#pragma unroll
                    for (int c = 0; c < kD / 8; ++c) dst[c] = src[c];
                } else {
                    const float inv1 = l_run > 0.f ? 1.0f / l_run : 0.f;
                    const float2 inv = make_float2(inv1, inv1);
#pragma unroll
                    for (int c = 0; c < kD / 8; ++c) {
                        float2 v4[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) v4[e] = __fmul2_rn(o_acc[4 * c + e], inv);
                        dst[c] = Vec16<__nv_bfloat16>::pack2(v4);
                    }
                }
            }
        }
        if (!ok) {
            if (args.status != nullptr) atomicExch(args.status, 1);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

PFN_cuTensorMapEncodeTiled_v12000 encode_fn() {
    static PFN_cuTensorMapEncodeTiled_v12000 fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult res;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &res) == cudaSuccess &&
            res == cudaDriverEntryPointSuccess) {
            fn = reinterpret_cast<PFN_cuTensorMapEncodeTiled_v12000>(p);
        } else {
            cudaGetLastError();
        }
    }
    return fn;
}

// bf16 tensor addressed as (d, row, head, batch) with element strides (1, sl, sh, sb); tiles of 128 rows x 64
bool make_tmap(CUtensorMap* map, const void* base, int64_t rows, int64_t heads, int64_t batch, int64_t sl, int64_t sh,
               int64_t sb) {
    PFN_cuTensorMapEncodeTiled_v12000 fn = encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[4] = {static_cast<cuuint64_t>(kD), static_cast<cuuint64_t>(rows), static_cast<cuuint64_t>(heads),
                                static_cast<cuuint64_t>(batch)};
    const cuuint64_t strides[3] = {static_cast<cuuint64_t>(sl) * 2, static_cast<cuuint64_t>(sh) * 2,
                                   static_cast<cuuint64_t>(sb > 0 ? sb : sl * rows) * 2};
    const cuuint32_t box[4] = {static_cast<cuuint32_t>(kD), static_cast<cuuint32_t>(kBN), 1, 1};
    const cuuint32_t elem[4] = {1, 1, 1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, elem,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

}  // namespace

bool attn_tc05_supported(const AttnArgs& a, int head_dim, int dtype) {
    return head_dim == kD && dtype == TB200_BF16 && a.key_valid == nullptr;
}

// total_rows: rows of the packed matrices (cu_rows given), ignored otherwise
int attn_tc05_forward(const AttnArgs& a, int max_lq, int64_t total_rows, int32_t* status, cudaStream_t stream) {
    const bool packed = a.cu_rows != nullptr;
    CUtensorMap tq, tk, tv;
    const int64_t q_rows = packed ? total_rows : a.Lq;
    const int64_t k_rows = packed ? total_rows : a.Lk;
    const int64_t nb = packed ? 1 : a.B;
    if (!make_tmap(&tq, a.q, q_rows, a.H, nb, a.q_sl, a.q_sh, packed ? 0 : a.q_sb) ||
        !make_tmap(&tk, a.k, k_rows, a.H, nb, a.k_sl, a.k_sh, packed ? 0 : a.k_sb) ||
        !make_tmap(&tv, a.v, k_rows, a.H, nb, a.v_sl, a.v_sh, packed ? 0 : a.v_sb))
        return TB200_ERR_DRIVER;
    const DeviceInfo& dev = device_info();
    const size_t smem = (1 + kSlots) * kTileBytes + 1024;
    static bool attr_set[64] = {};
    if (!attr_set[dev.index]) {
        cudaFuncSetAttribute(attn_tc05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        attr_set[dev.index] = true;
    }
    Tc05Args args{a, status};
    (void)max_lq;
    const int64_t items = static_cast<int64_t>((a.Lq + kBM - 1) / kBM) * a.H * a.B;
    int64_t grid = static_cast<int64_t>(dev.sm_count) * 2;  // persistent: two CTAs per SM
    if (grid > items) grid = items;
    attn_tc05_kernel<<<static_cast<unsigned>(grid), kThreads, smem, stream>>>(tq, tk, tv, args);
    count_launch();
    return launch_status();
}

}  // namespace tb200
