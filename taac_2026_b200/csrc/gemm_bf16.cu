// Grouped bf16 GEMM with a fused epilogue for sm_100a:
//     out[g] = act(a[g] x w[g]^T + bias[g]) (+ residual[g])        g = 0 .. groups - 1
// a: [groups, M, K], w: [groups, N, K] (the layout of stacked `nn.Linear` weights), out / residual:
// [groups, M, N], all bf16 and contiguous; bias: [groups, N] fp32.  These are the per-token projections and
// feed-forward layers of the non-sequence tokens: every token has its own weights, so the batch of one token is
// one group.  A library batched GEMM leaves the bias, the SiLU and the residual to further passes over the
// result; here they ride in the epilogue, and the result is written once.
//
// Two kernels share the file.  `gemm_bf16_pair_kernel` (further down) is the one that normally runs: clusters of
// two CTAs on 256 x 256 tiles with tcgen05 cta_group::2.  `gemm_bf16_kernel` is its single-CTA form, used for
// matrices of at most 128 rows and when TB200_GEMM_PAIR=0 is set in the environment (for comparison):
// one persistent CTA per SM walks the (group, row tile, column tile) list round-robin, column tiles fastest,
// so that the CTAs working side by side share the activation rows.  Roles in its CTA of 320 threads:
//   warp 0      TMA producer: ring of {A 128 x 64, W 256 x 64} bf16 tiles, 128-byte swizzle, 4 stages
//   warp 1      MMA issuer (one lane): tcgen05.mma kind::f16 128 x 256 x 16, the whole K range of a tile
//               accumulates in one of two 256-column TMEM buffers
//   warps 2..9  epilogue: a thread owns one row, reads 32 of its columns from TMEM per round, adds the bias, applies
//               the activation, adds the residual (read from global memory a round ahead) and writes bf16 into one
//               of two alternating 128-byte-swizzled 16 KB staging boxes that one thread hands to TMA; meanwhile the
//               tensor cores fill the other TMEM buffer with the next tile.
// Every wait on an mbarrier is bounded; a wait that gives up raises the status word and all roles drain out
// through the final barrier, where the TMEM allocation is released.
#include <cudaTypedefs.h>

#include <cstdlib>

#include "tb200_common.cuh"
#include "tb200_ptx.cuh"

namespace tb200 {
void count_launch();

namespace {

constexpr int kBM = 128;
constexpr int kBN = 256;
constexpr int kBKBytes = 128;            // 64 bf16 per stage: one 128-byte swizzle atom
constexpr int kStages = 4;
constexpr int kEpiWarps = 8;
constexpr int kEpiThreads = kEpiWarps * 32;
constexpr int kThreads = 64 + kEpiThreads;
constexpr uint32_t kABytes = kBM * kBKBytes;   // 16 KB
constexpr uint32_t kBBytes = kBN * kBKBytes;   // 32 KB
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kBoxBytes = kBM * 128;      // staging box: 128 rows x 64 bf16
constexpr int kBoxes = kBN * 2 / 128;          // 4 boxes per tile, sent one after the other
constexpr uint32_t kOutBytes = 2 * kBoxBytes;  // two boxes in shared memory: one is stored while the next is filled
constexpr uint32_t kTmemCols = 512;
constexpr size_t kSmemBytes = static_cast<size_t>(kStages) * kStageBytes + kOutBytes + 1024;

struct GArgs {
    const float* bias;      // [groups, N] or nullptr
    int32_t* status;
    int32_t groups, N, K;
    int64_t M;
    int32_t act;            // 0 = none, 1 = SiLU, 2 = SiLU-gated pairs (column c gates column c + 128 of its 256-column tile)
    int32_t has_residual;
};

// silu(x) = h * tanh(h) + h, h = x / 2 (the result is rounded to bf16)
__device__ __forceinline__ float2 silu2(float2 x) {
    const float2 h = __fmul2_rn(x, make_float2(0.5f, 0.5f));
    float2 t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t.x) : "f"(h.x));
    asm("tanh.approx.f32 %0, %1;" : "=f"(t.y) : "f"(h.y));
    return __ffma2_rn(h, t, h);
}

__global__ void __launch_bounds__(kThreads, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                 const __grid_constant__ CUtensorMap tmap_o, const GArgs g, const __nv_bfloat16* __restrict__ residual) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[kStages];
    __shared__ uint64_t empty_bar[kStages];
    __shared__ uint64_t tmem_full[2];
    __shared__ uint64_t tmem_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ __align__(16) float bias_s[kBN];
    __shared__ int s_abort;

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;
    uint8_t* out_s = smem + static_cast<size_t>(kStages) * kStageBytes;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int64_t m_tiles = (g.M + kBM - 1) / kBM;
    const int n_tiles = g.N / kBN;
    const int k_blocks = g.K / (kBKBytes / 2);
    const int64_t total = static_cast<int64_t>(g.groups) * m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], kEpiThreads);
        }
        s_abort = 0;
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

    // tile t -> column tile (fastest), row tile, group
    auto decode = [&](int64_t t, int& n0, int& m0, int& grp) {
        const int n = static_cast<int>(t % n_tiles);
        const int64_t rest = t / n_tiles;
        n0 = n * kBN;
        m0 = static_cast<int>(rest % m_tiles) * kBM;
        grp = static_cast<int>(rest / m_tiles);
    };

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tmap_a);
            tma_prefetch_desc(&tmap_w);
            uint32_t it = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < total && ok; t += gridDim.x) {
                int n0, m0, grp;
                decode(t, n0, m0, grp);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % kStages;
                    const uint32_t ph = (it / kStages) & 1;
                    if (!mbar_wait_sleep(&empty_bar[s], ph ^ 1) || *reinterpret_cast<volatile int*>(&s_abort)) {
                        ok = false;
                        break;
                    }
                    uint8_t* dst = ring + static_cast<size_t>(s) * kStageBytes;
                    mbar_expect_tx(&full_bar[s], kStageBytes);
                    tma_load_3d(dst, &tmap_a, kb * kBKBytes, m0, grp, &full_bar[s]);
                    tma_load_3d(dst + kABytes, &tmap_w, kb * kBKBytes, n0, grp, &full_bar[s]);
                }
            }
            if (!ok) {
                s_abort = 1;
                if (g.status != nullptr) atomicExch(g.status, 1);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0) {
            const uint32_t idesc = umma_idesc(1, 1, 0, 0, kBM, kBN);   // bf16 x bf16 -> f32, both K-major
            const uint64_t desc0 = umma_desc_sw128(0, 1024, 16);
            const uint32_t ring_lo = (smem_u32(ring) & 0x3FFFFu) >> 4;
            uint32_t s = 0, ph = 0, buf = 0, aph = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < total && ok; t += gridDim.x) {
                if (!mbar_wait_sleep(&tmem_empty[buf], aph ^ 1)) { ok = false; break; }
                const uint32_t d_tmem = tmem_base + buf * kBN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait_sleep(&full_bar[s], ph)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t a_lo = ring_lo + s * (kStageBytes >> 4);
                    const uint64_t da = desc0 + a_lo;
                    const uint64_t db = desc0 + a_lo + (kABytes >> 4);
#pragma unroll
                    for (int k = 0; k < kBKBytes / 32; ++k) mma_f16_ss(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    tc_commit(&empty_bar[s]);
                    if (++s == kStages) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (!ok) break;
                tc_commit(&tmem_full[buf]);
                aph ^= buf;
                buf ^= 1;
            }
            if (!ok) {
                s_abort = 1;
                if (g.status != nullptr) atomicExch(g.status, 1);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        const int et = threadIdx.x - 64;          // 0..255
        const bool gated = g.act == 2;
        const int sub = et >> 7;                  // columns [32 sub, 32 sub + 32) of a round's 64
        const int quarter = warp & 3;             // TMEM lanes [32 quarter, +32) are visible to this warp
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        const int swz = row_in_tile & 7;
        uint32_t tile_count = 0;
        uint32_t round_count = 0;                 // rounds so far: staging box round_count % 2
        bool ok = true;
        for (int64_t t = blockIdx.x; t < total; t += gridDim.x, ++tile_count) {
            int n0, m0, grp;
            decode(t, n0, m0, grp);
            const uint32_t buf = tile_count & 1;
            const uint32_t aph = (tile_count >> 1) & 1;
            bias_s[et] = g.bias != nullptr ? g.bias[static_cast<int64_t>(grp) * g.N + n0 + et] : 0.f;
            // residual pieces of round r: this thread's row, 32 columns = four 16-byte loads, one round ahead
            const int64_t row = static_cast<int64_t>(m0) + row_in_tile;
            const bool has_res = residual != nullptr && row < g.M;
            const uint4* res_row = reinterpret_cast<const uint4*>(
                residual + (static_cast<int64_t>(grp) * g.M + (has_res ? row : 0)) * g.N + n0 + sub * 32);
            uint4 res_cur[4], res_next[4];
#pragma unroll
            for (int q = 0; q < 4; ++q) res_cur[q] = has_res ? res_row[q] : make_uint4(0u, 0u, 0u, 0u);   // plain loads: `out` may be this tensor
            // A thread whose wait gives up stops waiting but keeps walking the tile list, so that it still meets
            // every named barrier the other epilogue threads sit in; what it writes is garbage and the status
            // word says so.
            if (ok && !mbar_wait_sleep(&tmem_full[buf], aph)) ok = false;
            tc_fence_after_sync();
            const int n_rounds = gated ? kBoxes / 2 : kBoxes;   // gated: 128 gate + 128 value columns -> 128 outputs
#pragma unroll 1
            for (int r = 0; r < n_rounds; ++r, ++round_count) {
                const int col = r * 64 + sub * 32;       // first of this thread's 32 columns in the tile
                uint8_t* box = out_s + (round_count & 1) * kBoxBytes;
                if (r + 1 < n_rounds) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) res_next[q] = has_res ? res_row[(r + 1) * 8 + q] : make_uint4(0u, 0u, 0u, 0u);
                }
                uint32_t acc[32], accv[32];
                tmem_ld_2x16(tmem_base + buf * kBN + lane_addr + col, acc);
                if (gated) tmem_ld_2x16(tmem_base + buf * kBN + lane_addr + 128 + col, accv);
                if (et == 0) bulk_wait_read<1>();   // the store that used this box two rounds ago has read it
                asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
                tc_wait_ld(acc);
                if (gated) tc_wait_ld(accv);   // no second wait in hardware terms; it keeps the uses of accv below the wait
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    const float4 b0 = *reinterpret_cast<const float4*>(bias_s + col + q * 8);
                    const float4 b1 = *reinterpret_cast<const float4*>(bias_s + col + q * 8 + 4);
                    float2 v[4];
                    v[0] = __fadd2_rn(make_float2(__uint_as_float(acc[8 * q + 0]), __uint_as_float(acc[8 * q + 1])), make_float2(b0.x, b0.y));
                    v[1] = __fadd2_rn(make_float2(__uint_as_float(acc[8 * q + 2]), __uint_as_float(acc[8 * q + 3])), make_float2(b0.z, b0.w));
                    v[2] = __fadd2_rn(make_float2(__uint_as_float(acc[8 * q + 4]), __uint_as_float(acc[8 * q + 5])), make_float2(b1.x, b1.y));
                    v[3] = __fadd2_rn(make_float2(__uint_as_float(acc[8 * q + 6]), __uint_as_float(acc[8 * q + 7])), make_float2(b1.z, b1.w));
                    if (g.act >= 1) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[e] = silu2(v[e]);
                    }
                    if (gated) {   // silu(gate) * value, the value columns sit 128 further right in the accumulator
                        const float4 c0 = *reinterpret_cast<const float4*>(bias_s + 128 + col + q * 8);
                        const float4 c1 = *reinterpret_cast<const float4*>(bias_s + 128 + col + q * 8 + 4);
                        v[0] = __fmul2_rn(v[0], __fadd2_rn(make_float2(__uint_as_float(accv[8 * q + 0]), __uint_as_float(accv[8 * q + 1])), make_float2(c0.x, c0.y)));
                        v[1] = __fmul2_rn(v[1], __fadd2_rn(make_float2(__uint_as_float(accv[8 * q + 2]), __uint_as_float(accv[8 * q + 3])), make_float2(c0.z, c0.w)));
                        v[2] = __fmul2_rn(v[2], __fadd2_rn(make_float2(__uint_as_float(accv[8 * q + 4]), __uint_as_float(accv[8 * q + 5])), make_float2(c1.x, c1.y)));
                        v[3] = __fmul2_rn(v[3], __fadd2_rn(make_float2(__uint_as_float(accv[8 * q + 6]), __uint_as_float(accv[8 * q + 7])), make_float2(c1.z, c1.w)));
                    }
                    if (residual != nullptr) {
                        float2 rr[4];
                        Vec16<__nv_bfloat16>::unpack2(res_cur[q], rr);
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[e] = __fadd2_rn(v[e], rr[e]);
                    }
                    *reinterpret_cast<uint4*>(box + row_in_tile * 128 + (((sub * 4 + q) ^ swz) << 4)) = Vec16<__nv_bfloat16>::pack2(v);
                }
                if (r == n_rounds - 1) {   // every column of this buffer has been read: the tensor cores may reuse it
                    tc_fence_before_sync();
                    mbar_arrive(&tmem_empty[buf]);
                }
                fence_proxy_async_smem();
                asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
                if (et == 0) {
                    tma_store_3d(&tmap_o, box, (gated ? n0 : 2 * n0) + r * 128, m0, grp);
                    bulk_commit();
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) res_cur[q] = res_next[q];
            }
        }
        if (et == 0) bulk_wait<0>();
        if (!ok) {
            s_abort = 1;
            if (g.status != nullptr) atomicExch(g.status, 1);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------------------------------------
// CTA-pair variant (cluster of two CTAs, tcgen05 cta_group::2).  A pair owns a 256 x 256 output tile: each CTA
// loads its own 128 rows of A and one half (128 rows) of the weight tile, the leader (even rank) issues
// 256 x 256 x 16 MMAs that read A from each CTA's own shared memory and the weight halves from both, and each
// CTA's TMEM receives its 128 rows.  A stage is then 32 KB per CTA for the same 512 cycles of tensor-core time,
// so six stages fit where the single-CTA kernel has four: the ring holds 3072 cycles of work, more than the
// round trip that the K loop otherwise waits for.  Barriers: the "full" barriers live in the leader and count
// the bytes of both CTAs' loads; "empty" and "accumulator full" are signalled in both CTAs by multicast
// commits; "accumulator empty" collects one arrival per epilogue warp of both CTAs in the leader.
// Epilogue: eight warps per CTA, two per TMEM lane quarter (one takes the even, one the odd 64-column boxes of
// its 32 rows).  A warp is self-contained: one lane polls the "accumulator full" barrier and broadcasts the
// outcome, the warp reads 16 columns per thread and round, arrives on "accumulator empty" right after its last
// tcgen05.ld (the MMAs of the next tile start while the values are still being converted), and sends its own
// 32-row x 128-byte box to TMA from a private 4 KB staging tile: no block-wide barrier anywhere in the epilogue.
// ------------------------------------------------------------------------------------------------
constexpr int kStagesP = 6;
constexpr int kEpiWarpsP = 8;                  // two warps per TMEM lane quarter, each with a staging box and TMA stores of its own
constexpr int kEpiThreadsP = kEpiWarpsP * 32;
constexpr int kThreadsP = 64 + kEpiThreadsP;
constexpr uint32_t kBHalfBytes = kBBytes / 2;                 // 16 KB: this CTA's half of the weight tile
constexpr uint32_t kStagePBytes = kABytes + kBHalfBytes;      // 32 KB
constexpr uint32_t kWarpBoxBytes = 32 * 128;                  // one epilogue warp's staging box: 32 rows x 64 bf16
constexpr size_t kSmemPBytes = static_cast<size_t>(kStagesP) * kStagePBytes + kEpiWarpsP * kWarpBoxBytes + 1024;
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;                   // shared::cluster address of the pair's even CTA

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_3d_pair(void* smem_dst, const CUtensorMap* m, int32_t c0, int32_t c1, int32_t c2,
                                                 uint64_t* leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.3d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], "
        "[%2];" ::"r"(smem_u32(smem_dst)),
        "l"(m), "r"(smem_u32(leader_bar) & kPeerMask), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void mma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// arrives on the barrier at this shared-memory offset in BOTH CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;" ::"r"(
                     smem_u32(bar)),
                 "h"(static_cast<uint16_t>(3))
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive_leader(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cluster.b64 _, [%0];" ::"r"(smem_u32(bar) & kPeerMask) : "memory");
}

template <bool GATED, bool RES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreadsP, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_w,
                      const __grid_constant__ CUtensorMap tmap_o, const GArgs g, const __nv_bfloat16* __restrict__ residual) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[kStagesP];     // used in the leader only
    __shared__ uint64_t empty_bar[kStagesP];
    __shared__ uint64_t tmem_full[2];
    __shared__ uint64_t tmem_empty[2];          // used in the leader only
    __shared__ uint32_t tmem_base_slot;
    __shared__ int s_abort;

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* ring = smem;
    uint8_t* out_s = smem + static_cast<size_t>(kStagesP) * kStagePBytes;
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();       // 0 = leader
    const int64_t pair = blockIdx.x >> 1;
    const int64_t n_pairs = gridDim.x >> 1;

    const int64_t m_tiles = (g.M + 2 * kBM - 1) / (2 * kBM);
    const int n_tiles = g.N / kBN;
    const int k_blocks = g.K / (kBKBytes / 2);
    const int64_t total = static_cast<int64_t>(g.groups) * m_tiles * n_tiles;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kStagesP; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            mbar_init(&tmem_full[b], 1);
            mbar_init(&tmem_empty[b], 2 * kEpiWarpsP);
        }
        s_abort = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&tmem_base_slot)), "r"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                          // both CTAs' barriers exist before anything is signalled remotely
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    auto decode = [&](int64_t t, int& n0, int& m0, int& grp) {
        const int n = static_cast<int>(t % n_tiles);
        const int64_t rest = t / n_tiles;
        n0 = n * kBN;
        m0 = static_cast<int>(rest % m_tiles) * 2 * kBM + static_cast<int>(rank) * kBM;   // this CTA's 128 rows
        grp = static_cast<int>(rest / m_tiles);
    };

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer (both CTAs)
        if (lane == 0) {
            tma_prefetch_desc(&tmap_a);
            tma_prefetch_desc(&tmap_w);
            uint32_t it = 0;
            bool ok = true;
            for (int64_t t = pair; t < total && ok; t += n_pairs) {
                int n0, m0, grp;
                decode(t, n0, m0, grp);
                for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                    const uint32_t s = it % kStagesP;
                    const uint32_t ph = (it / kStagesP) & 1;
                    if (!mbar_wait_sleep(&empty_bar[s], ph ^ 1) || *reinterpret_cast<volatile int*>(&s_abort)) {
                        ok = false;
                        break;
                    }
                    uint8_t* dst = ring + static_cast<size_t>(s) * kStagePBytes;
                    if (rank == 0) mbar_expect_tx(&full_bar[s], 2 * kStagePBytes);   // the bytes of both CTAs
                    tma_load_3d_pair(dst, &tmap_a, kb * kBKBytes, m0, grp, &full_bar[s]);
                    tma_load_3d_pair(dst + kABytes, &tmap_w, kb * kBKBytes, n0 + static_cast<int>(rank) * (kBN / 2), grp, &full_bar[s]);
                }
            }
            if (!ok) {
                s_abort = 1;
                if (g.status != nullptr) atomicExch(g.status, 1);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (leader only)
        if (lane == 0 && rank == 0) {
            const uint32_t idesc = umma_idesc(1, 1, 0, 0, 2 * kBM, kBN);
            const uint64_t desc0 = umma_desc_sw128(0, 1024, 16);
            const uint32_t ring_lo = (smem_u32(ring) & 0x3FFFFu) >> 4;
            uint32_t s = 0, ph = 0, buf = 0, aph = 0;
            bool ok = true;
            for (int64_t t = pair; t < total && ok; t += n_pairs) {
                if (!mbar_wait_sleep(&tmem_empty[buf], aph ^ 1)) { ok = false; break; }
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + buf * kBN;
                for (int kb = 0; kb < k_blocks; ++kb) {
                    if (!mbar_wait_sleep(&full_bar[s], ph)) { ok = false; break; }
                    tc_fence_after_sync();
                    const uint32_t a_lo = ring_lo + s * (kStagePBytes >> 4);
                    const uint64_t da = desc0 + a_lo;
                    const uint64_t db = desc0 + a_lo + (kABytes >> 4);
#pragma unroll
                    for (int k = 0; k < kBKBytes / 32; ++k) mma_f16_ss_pair(d_tmem, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                    tc_commit_pair(&empty_bar[s]);
                    if (++s == kStagesP) {
                        s = 0;
                        ph ^= 1;
                    }
                }
                if (!ok) break;
                tc_commit_pair(&tmem_full[buf]);
                aph ^= buf;
                buf ^= 1;
            }
            if (!ok) {
                s_abort = 1;
                if (g.status != nullptr) atomicExch(g.status, 1);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
        // Every warp works alone: it owns the 32 rows of its TMEM lane quarter and 128 of the tile's 256 columns, and
        // sends them out as two units of 64 columns: 32 columns at a time from TMEM to registers, bias / activation /
        // residual, bf16 into its private 4 KB staging box (32 rows x 128 bytes, 128-byte swizzle), one TMA store per
        // unit.  No barrier spans the CTA, so no warp waits for the slowest one or for another warp's store, and the
        // accumulator buffer is handed back as soon as the warp's last load has landed in registers.  Boxes are 128
        // bytes wide on purpose: the TMA unit works row by row, and narrower boxes (64-byte rows, 16 warps) doubled
        // its store requests and slowed the long-K shapes by a tenth, because the loads of the K loop queue behind them.
        const int ew = warp - 2;                  // 0..7
        constexpr bool gated = GATED;
        const int half = ew >> 2;                 // non-gated: columns [128 half, +128); gated: outputs [64 half, +64)
        const int quarter = warp & 3;             // TMEM lanes [32 quarter, +32) are the ones this warp may read
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        uint8_t* box = out_s + ew * kWarpBoxBytes;
        const int swz = lane & 7;                 // 128-byte swizzle: 16-byte piece ^ (row % 8)
        constexpr int kUnits = gated ? 1 : 2;
        uint32_t tile_count = 0;
        bool ok = true;
        for (int64_t t = pair; t < total; t += n_pairs, ++tile_count) {
            int n0, m0, grp;
            decode(t, n0, m0, grp);
            const uint32_t buf = tile_count & 1;
            const uint32_t aph = (tile_count >> 1) & 1;
            const int64_t row = static_cast<int64_t>(m0) + row_in_tile;
            const bool has_res = RES && row < g.M;
            const float* bias_t = g.bias != nullptr ? g.bias + static_cast<int64_t>(grp) * g.N + n0 : nullptr;
            // this thread's residual row: plain loads (`out` may be this tensor), a 32-column piece ahead of its use
            const uint4* res_row = RES ? reinterpret_cast<const uint4*>(
                residual + (static_cast<int64_t>(grp) * g.M + (has_res ? row : 0)) * g.N + n0 + half * 128) : nullptr;
            uint4 res[RES ? 4 : 1];
            if (RES) {
#pragma unroll
                for (int q = 0; q < 4; ++q) res[RES ? q : 0] = has_res ? res_row[q] : make_uint4(0u, 0u, 0u, 0u);
            }
            // A warp whose wait gives up stops waiting but keeps walking the tile list (it still arrives on the
            // accumulator barrier, so the other roles are not held up by it); its output is garbage, the status word says so.
            if (ok) {   // one lane polls, the warp follows
                int passed = 1;
                if (lane == 0) passed = mbar_wait_sleep(&tmem_full[buf], aph) ? 1 : 0;
                if (__shfl_sync(0xffffffffu, passed, 0) == 0) ok = false;
            }
            tc_fence_after_sync();
#pragma unroll 1
            for (int piece = 0; piece < 2 * kUnits; ++piece) {       // 32 accumulator columns per piece, two pieces per store
                const int sub = piece & 1;
                const int col = gated ? half * 64 + piece * 32 : half * 128 + piece * 32;   // first accumulator column
                uint32_t acc[32], accv[gated ? 32 : 1];
                tmem_ld_2x16(tmem_base + buf * kBN + lane_addr + col, acc);
                if (gated) tmem_ld_2x16(tmem_base + buf * kBN + lane_addr + 128 + col, *reinterpret_cast<uint32_t (*)[32]>(&accv[0]));
                if (sub == 0 && lane == 0) bulk_wait_read<0>();     // this warp's previous store has read the box
                tc_wait_ld(acc);
                if (gated) tc_wait_ld(*reinterpret_cast<uint32_t (*)[32]>(&accv[0]));
                if (piece == 2 * kUnits - 1) {          // the warp holds its share of the buffer in registers: hand it back
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_leader(&tmem_empty[buf]);
                } else {
                    __syncwarp();
                }
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;
                    if (bias_t != nullptr) {
                        b0 = __ldg(reinterpret_cast<const float4*>(bias_t + col + q * 8));
                        b1 = __ldg(reinterpret_cast<const float4*>(bias_t + col + q * 8 + 4));
                    }
                    float2 v[4];
                    v[0] = __fadd2_rn(make_float2(__uint_as_float(acc[8 * q + 0]), __uint_as_float(acc[8 * q + 1])), make_float2(b0.x, b0.y));
                    v[1] = __fadd2_rn(make_float2(__uint_as_float(acc[8 * q + 2]), __uint_as_float(acc[8 * q + 3])), make_float2(b0.z, b0.w));
                    v[2] = __fadd2_rn(make_float2(__uint_as_float(acc[8 * q + 4]), __uint_as_float(acc[8 * q + 5])), make_float2(b1.x, b1.y));
                    v[3] = __fadd2_rn(make_float2(__uint_as_float(acc[8 * q + 6]), __uint_as_float(acc[8 * q + 7])), make_float2(b1.z, b1.w));
                    if (g.act >= 1) {
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[e] = silu2(v[e]);
                    }
                    if (gated) {   // silu(gate) * value, the value columns sit 128 further right in the accumulator
                        float4 c0 = make_float4(0.f, 0.f, 0.f, 0.f), c1 = c0;
                        if (bias_t != nullptr) {
                            c0 = __ldg(reinterpret_cast<const float4*>(bias_t + 128 + col + q * 8));
                            c1 = __ldg(reinterpret_cast<const float4*>(bias_t + 128 + col + q * 8 + 4));
                        }
                        constexpr int G = gated ? 1 : 0;   // keeps the indices inside accv[1] in the non-gated instantiation
                        v[0] = __fmul2_rn(v[0], __fadd2_rn(make_float2(__uint_as_float(accv[G * (8 * q + 0)]), __uint_as_float(accv[G * (8 * q + 1)])), make_float2(c0.x, c0.y)));
                        v[1] = __fmul2_rn(v[1], __fadd2_rn(make_float2(__uint_as_float(accv[G * (8 * q + 2)]), __uint_as_float(accv[G * (8 * q + 3)])), make_float2(c0.z, c0.w)));
                        v[2] = __fmul2_rn(v[2], __fadd2_rn(make_float2(__uint_as_float(accv[G * (8 * q + 4)]), __uint_as_float(accv[G * (8 * q + 5)])), make_float2(c1.x, c1.y)));
                        v[3] = __fmul2_rn(v[3], __fadd2_rn(make_float2(__uint_as_float(accv[G * (8 * q + 6)]), __uint_as_float(accv[G * (8 * q + 7)])), make_float2(c1.z, c1.w)));
                    }
                    if (RES) {
                        float2 rr[4];
                        Vec16<__nv_bfloat16>::unpack2(res[RES ? q : 0], rr);
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[e] = __fadd2_rn(v[e], rr[e]);
                    }
                    *reinterpret_cast<uint4*>(box + lane * 128 + (((sub * 4 + q) ^ swz) << 4)) = Vec16<__nv_bfloat16>::pack2(v);
                }
                if (RES && piece + 1 < 2 * kUnits) {   // the next piece's residual columns
#pragma unroll
                    for (int q = 0; q < 4; ++q) res[RES ? q : 0] = has_res ? res_row[(piece + 1) * 4 + q] : make_uint4(0u, 0u, 0u, 0u);
                }
                if (sub == 1) {
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        const int32_t x_bytes = gated ? n0 + half * 128 : 2 * n0 + half * 256 + (piece >> 1) * 128;
                        const int32_t y = m0 + quarter * 32;
                        if (y < g.M) tma_store_3d(&tmap_o, box, x_bytes, y, grp);   // rows past M are clipped by the tensor map
                        bulk_commit();
                    }
                }
            }
        }
        if (lane == 0) bulk_wait<0>();            // the last store must have left shared memory before the CTA ends
        if (!ok) {
            s_abort = 1;
            if (g.status != nullptr) atomicExch(g.status, 1);
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                          // the peer may still read this CTA's shared memory or signal its barriers
    if (warp == 1) {
        tc_fence_after_sync();
        asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
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

// [groups, rows, row_bytes] bytes, boxes of box_rows x box_bytes (128 or 64) inside one group, swizzle of the box width
bool make_tmap3(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint64_t groups, uint32_t box_rows,
                uint32_t box_bytes = 128) {
    PFN_cuTensorMapEncodeTiled_v12000 fn = encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[3] = {row_bytes, rows, groups};
    const cuuint64_t strides[2] = {row_bytes, row_bytes * rows};
    const cuuint32_t box[3] = {box_bytes, box_rows, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, box_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_gemm_bf16_grouped(const void* a, const void* w, const float* bias, const void* residual, void* out,
                                       int32_t groups, int64_t M, int32_t N, int32_t K, int32_t act,
                                       int32_t* status_word, void* stream) {
    using namespace tb200;
    if (groups < 0 || M < 0 || N < kBN || N % kBN != 0 || K < 64 || K % 64 != 0) return TB200_ERR_SHAPE;
    if (act < 0 || act > 2 || (act == 2 && residual != nullptr)) return TB200_ERR_UNSUPPORTED;
    if (groups == 0 || M == 0) return TB200_OK;
    if (a == nullptr || w == nullptr || out == nullptr) return TB200_ERR_NULL;
    if (!aligned16(a) || !aligned16(w) || !aligned16(out) || (residual != nullptr && !aligned16(residual)) ||
        (bias != nullptr && (reinterpret_cast<uintptr_t>(bias) & 3) != 0))
        return TB200_ERR_ALIGN;
    if (M > 0x7FFFFF00ll || static_cast<int64_t>(groups) * ((M + kBM - 1) / kBM) * (N / kBN) > 0x7FFFFFFFll) return TB200_ERR_SHAPE;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    CUtensorMap ta, tw, to;
    const uint64_t ug = static_cast<uint64_t>(groups), um = static_cast<uint64_t>(M);
    if (!make_tmap3(&ta, a, 2ull * K, um, ug, kBM) || !make_tmap3(&tw, w, 2ull * K, static_cast<uint64_t>(N), ug, kBN) ||
        !make_tmap3(&to, out, act == 2 ? static_cast<uint64_t>(N) : 2ull * N, um, ug, kBM))
        return TB200_ERR_DRIVER;
    GArgs g{};
    g.bias = bias;
    g.status = status_word;
    g.groups = groups;
    g.N = N;
    g.K = K;
    g.M = M;
    g.act = act;
    g.has_residual = residual != nullptr ? 1 : 0;
    const DeviceInfo& dev = device_info();
    static bool attr_set[64] = {};
    if (!attr_set[dev.index]) {
        cudaFuncSetAttribute(gemm_bf16_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemBytes));
        attr_set[dev.index] = true;
    }
    // CTA pairs by default; TB200_GEMM_PAIR=0 in the environment selects the single-CTA kernel (for comparison)
    static const bool use_pair = []() { const char* e = getenv("TB200_GEMM_PAIR"); return e == nullptr || e[0] != '0'; }();
    if (use_pair && M > kBM) {
        static bool pair_attr[64] = {};
        if (!pair_attr[dev.index]) {
            cudaFuncSetAttribute(gemm_bf16_pair_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemPBytes));
            cudaFuncSetAttribute(gemm_bf16_pair_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemPBytes));
            cudaFuncSetAttribute(gemm_bf16_pair_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(kSmemPBytes));
            pair_attr[dev.index] = true;
        }
        CUtensorMap twh, tow;
        if (!make_tmap3(&twh, w, 2ull * K, static_cast<uint64_t>(N), ug, kBN / 2)) return TB200_ERR_DRIVER;
        if (!make_tmap3(&tow, out, act == 2 ? static_cast<uint64_t>(N) : 2ull * N, um, ug, 32)) return TB200_ERR_DRIVER;
        const int64_t tiles = static_cast<int64_t>(groups) * ((M + 2 * kBM - 1) / (2 * kBM)) * (N / kBN);
        int64_t pairs = dev.sm_count / 2;
        if (pairs > tiles) pairs = tiles;
        const unsigned grid = static_cast<unsigned>(2 * pairs);
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        const __nv_bfloat16* res = static_cast<const __nv_bfloat16*>(residual);
        if (act == 2)
            gemm_bf16_pair_kernel<true, false><<<grid, kThreadsP, kSmemPBytes, st>>>(ta, twh, tow, g, res);
        else if (residual != nullptr)
            gemm_bf16_pair_kernel<false, true><<<grid, kThreadsP, kSmemPBytes, st>>>(ta, twh, tow, g, res);
        else
            gemm_bf16_pair_kernel<false, false><<<grid, kThreadsP, kSmemPBytes, st>>>(ta, twh, tow, g, res);
        count_launch();
        return launch_status();
    }
    const int64_t total = static_cast<int64_t>(groups) * ((M + kBM - 1) / kBM) * (N / kBN);
    const int64_t grid = total < dev.sm_count ? total : dev.sm_count;
    gemm_bf16_kernel<<<static_cast<unsigned>(grid), kThreads, kSmemBytes, static_cast<cudaStream_t>(stream)>>>(
        ta, tw, to, g, static_cast<const __nv_bfloat16*>(residual));
    count_launch();
    return launch_status();
}
