// FP8 (e4m3) block-scaled FFN for sm_100a: activation quantisation and the two GEMMs, with the
// dequantisation scales, bias, SiLU / SiLU-gating and the re-quantisation of the hidden activation
// fused into the GEMM epilogues.
//
// Scales are fp32 amax scales — one per 1 x 128 block of an activation row and one per 128 x 128
// block of a weight — so every 128-wide K block has its own scale pair.  The tensor cores therefore
// produce one partial product per K block in TMEM (tcgen05.mma kind::f8f6f4, 128 x 256 x 32 per
// instruction, operands staged by TMA in 128-byte-swizzled shared memory), and the epilogue warps
// promote it into fp32 register accumulators with the block's scale while the tensor cores already
// work on the next K block (two TMEM accumulator buffers of 256 columns).
//
// Roles in a CTA of 576 threads (persistent, one CTA per SM, static round-robin over output tiles):
//   warp 0       TMA producer: ring of {A 128 x 128 B, B 256 x 128 B} tiles (3 to 4 stages)
//   warp 1       MMA issuer (one elected lane), owner of the TMEM allocation
//   warps 2..17  promotion + epilogue: each thread owns one output row and 64 of the 256 columns
//                (four warps per TMEM lane quarter, so that four warps per scheduler hide each
//                other's tcgen05.ld and MUFU latencies; the per-element instruction allowance at K = 512
//                is only about eight issue slots, hence packed fp32x2 math and a tanh-based SiLU)
// The output tile leaves through shared memory: every epilogue thread writes its 16-byte pieces into a
// 128-byte-swizzled staging tile and one thread hands the tile to TMA, so global memory sees full rows of
// the tile instead of one 32-byte sector per lane; the residual tile of the linear mode arrives the same
// way, fetched by TMA while the K loop runs.
// Every wait on an mbarrier is bounded; a wait that gives up raises the status word and all roles
// drain out through the same final barrier, where the TMEM allocation is released.
#include <cuda_fp8.h>
#include <cudaTypedefs.h>

#include <mutex>

#include "tb200_common.cuh"
#include "tb200_ptx.cuh"

namespace tb200 {
void count_launch();

namespace {

constexpr int kBM = 128;          // output rows per tile
constexpr int kBN = 256;          // output columns per tile
constexpr int kBK = 128;          // K bytes (= e4m3 elements) per stage: one 128-byte swizzle atom
constexpr int kThreads = 576;
constexpr int kEpiThreads = 512;
constexpr uint32_t kABytes = kBM * kBK;  // 16 KB
constexpr uint32_t kBBytes = kBN * kBK;  // 32 KB
constexpr uint32_t kStageBytes = kABytes + kBBytes;
constexpr uint32_t kTmemCols = 512;      // two 256-column fp32 accumulator buffers

enum Mode : int {
    kSwiGLU = 0,  // columns = [128 gate | 128 up] of one hidden block -> fp8 hidden + 1x128 scales
    kSiLU = 1,    // hidden = silu(acc + bias)                          -> fp8 hidden + 1x128 scales
    kLinear = 2,  // y = acc + bias (+ residual)                        -> bf16
};

struct GemmArgs {
    const float* sa;     // [M, K / 128] activation scales
    const float* sb;     // [N / 128, K / 128] weight scales
    const float* bias;   // [N] fp32 or nullptr (for kSwiGLU in the tile's interleaved column order)
    const __nv_bfloat16* residual;  // [M, N] or nullptr (kLinear only)
    void* out;           // kLinear: bf16 [M, N]; else e4m3 [M, N_hidden]
    float* out_scale;    // [M, N_hidden / 128] (quantising modes)
    int32_t* status;     // device word: set to 1 when a wait gave up (may be nullptr)
    int64_t M;
    int32_t N;           // GEMM columns (kSwiGLU: 2 * hidden)
    int32_t K;
    int32_t out_ld;      // row pitch of `out` in elements
};

// silu(x) = x * sigmoid(x) = h * tanh(h) + h with h = x / 2: one MUFU and two FMA-pipe instructions.
// tanh.approx has about 11 bits of accuracy, far below the 3-bit mantissa of the e4m3 result.  (The packed
// tanh.approx.f16x2 halves the MUFU count but was measured no faster here, and its absolute error near -1
// shows in the hidden activation of strongly negative inputs.)
__device__ __forceinline__ float silu(float x) {
    const float h = 0.5f * x;
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
    return fmaf(h, t, h);
}

// 64 fp32 -> 64 e4m3 bytes (as 16 words) with q = x * inv_scale, round-to-nearest, saturating
__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// Work distribution: a CTA keeps ONE column tile (256 weight rows) for its whole life and walks down
// the row tiles, so the weight tile, its scales and the bias are fetched once per CTA.  With
// n_tiles <= gridDim.x, CTA c owns column tile c % n_tiles and row tiles j, j + G, ... (j = c / n_tiles,
// G = gridDim.x / n_tiles); the n_tiles CTAs that share j read the same activation rows at about the
// same time, so those rows come from HBM once.  If K <= 512 the weight tile stays resident in shared
// memory (B_RES) and only the activation tiles stream through the ring.
struct Schedule {
    int n_first, n_step, j, G;
    bool active;
};
__device__ __forceinline__ Schedule make_schedule(int n_tiles) {
    Schedule sc;
    const int c = blockIdx.x;
    const int grid = gridDim.x;
    if (n_tiles <= grid) {
        sc.G = grid / n_tiles;
        sc.n_first = c % n_tiles;
        sc.j = c / n_tiles;
        sc.n_step = 0x40000000;  // a single column tile per CTA
        sc.active = sc.j < sc.G;
    } else {
        sc.G = 1;
        sc.j = 0;
        sc.n_first = c;
        sc.n_step = grid;
        sc.active = true;
    }
    return sc;
}

constexpr int kMaxStages = 5;
constexpr uint32_t kOutBoxBytes = kBM * 128;   // one staging box: 128 rows x 128 bytes, 128-byte swizzle

// Shared-memory plan per instantiation.  Static shared memory takes about 6 KB, so tiles + staging stay
// at or below 208 KB.  B_RES keeps up to four 32 KB weight K blocks resident.
template <int MODE, bool B_RES>
struct Plan {
    static constexpr int kOutBoxes = MODE == kSwiGLU ? 1 : (MODE == kSiLU ? 2 : 4);
    static constexpr uint32_t kOutBytes = kOutBoxes * kOutBoxBytes;
    static constexpr int kStagesN = B_RES ? (MODE == kSwiGLU ? 4 : 3) : (MODE == kSwiGLU ? 4 : 3);
    static constexpr uint32_t kStageBytesN = B_RES ? kABytes : kStageBytes;
    static constexpr size_t tiles_bytes(int k_blocks) {
        return (B_RES ? static_cast<size_t>(k_blocks) * kBBytes : 0) + static_cast<size_t>(kStagesN) * kStageBytesN + kOutBytes;
    }
};
constexpr int kMaxKBlocks = 64;   // K <= 8192

template <int MODE, bool B_RES>
__global__ void __launch_bounds__(kThreads, 1)
ffn_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                const __grid_constant__ CUtensorMap tmap_o, const __grid_constant__ CUtensorMap tmap_r, const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[kMaxStages];
    __shared__ uint64_t empty_bar[kMaxStages];
    __shared__ uint64_t b_full;
    __shared__ uint64_t res_full;   // residual tile of the linear mode has landed in the staging tile
    __shared__ uint64_t tmem_full[2];
    __shared__ uint64_t tmem_empty[2];
    __shared__ uint32_t tmem_base_slot;
    __shared__ __align__(16) float bias_s[kBN];
    __shared__ float sb_s[2][kMaxKBlocks];
    __shared__ float amax_xchg[2][4][kBM];
    __shared__ int s_abort;

    // tiles need 1024-byte alignment for the 128-byte swizzle pattern
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int64_t m_tiles = (g.M + kBM - 1) / kBM;
    const int n_tiles = g.N / kBN;
    const int k_blocks = g.K / kBK;
    using P = Plan<MODE, B_RES>;
    constexpr int STAGES = P::kStagesN;
    constexpr uint32_t STAGE_BYTES = P::kStageBytesN;
    uint8_t* b_res = smem;                                              // [k_blocks][kBBytes] when B_RES
    uint8_t* ring = B_RES ? smem + static_cast<size_t>(k_blocks) * kBBytes : smem;
    uint8_t* out_s = ring + static_cast<size_t>(STAGES) * STAGE_BYTES;    // staging tile: kOutBoxes boxes of 16 KB
    const Schedule sc = make_schedule(n_tiles);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&b_full, 1);
        mbar_init(&res_full, 1);
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

    if (warp == 0) {
        // ---------------------------------------------------------------- TMA producer
        if (lane == 0 && sc.active) {
            tma_prefetch_desc(&tmap_a);
            tma_prefetch_desc(&tmap_b);
            uint32_t it = 0;
            bool ok = true;
            for (int n = sc.n_first; n < n_tiles && ok; n += sc.n_step) {
                const int n0 = n * kBN;
                if (B_RES) {
                    if (it > 0) {  // the previous column tile's MMAs must have finished reading b_res
                        const uint32_t last = it - 1;
                        if (!mbar_wait_sleep(&empty_bar[last % STAGES], (last / STAGES) & 1)) { ok = false; break; }
                    }
                    mbar_expect_tx(&b_full, static_cast<uint32_t>(k_blocks) * kBBytes);
                    for (int kb = 0; kb < k_blocks; ++kb)
                        tma_load_2d(b_res + static_cast<size_t>(kb) * kBBytes, &tmap_b, kb * kBK, n0, &b_full);
                }
                for (int64_t m = sc.j; m < m_tiles && ok; m += sc.G) {
                    const int m0 = static_cast<int>(m) * kBM;
                    for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                        const uint32_t s = it % STAGES;
                        const uint32_t ph = (it / STAGES) & 1;
                        if (!mbar_wait_sleep(&empty_bar[s], ph ^ 1) || *reinterpret_cast<volatile int*>(&s_abort)) {
                            ok = false;
                            break;
                        }
                        uint8_t* a_dst = ring + static_cast<size_t>(s) * STAGE_BYTES;
                        mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                        tma_load_2d(a_dst, &tmap_a, kb * kBK, m0, &full_bar[s]);
                        if (!B_RES) tma_load_2d(a_dst + kABytes, &tmap_b, kb * kBK, n0, &full_bar[s]);
                    }
                }
            }
            if (!ok) {
                s_abort = 1;
                if (g.status != nullptr) atomicExch(g.status, 1);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer
        if (lane == 0 && sc.active) {
            const uint32_t idesc = umma_idesc(0, 0, 0, 0, kBM, kBN);  // e4m3 x e4m3 -> f32, both K-major
            // This one thread sets the pace of the tensor pipe, so its loop carries no division and builds each
            // descriptor with one add: the start-address field counts 16-byte units, a 32-byte K step adds 2.
            const uint64_t desc0 = umma_desc_sw128(0, 1024, 16);
            const uint32_t ring_lo = (smem_u32(ring) & 0x3FFFFu) >> 4;
            const uint32_t bres_lo = B_RES ? (smem_u32(b_res) & 0x3FFFFu) >> 4 : 0u;
            uint32_t s = 0, ph = 0, buf = 0, aph = 0, b_phase = 0;
            bool ok = true;
            for (int n = sc.n_first; n < n_tiles && ok; n += sc.n_step) {
                if (B_RES) {
                    if (!mbar_wait_sleep(&b_full, b_phase)) { ok = false; break; }
                    b_phase ^= 1;
                }
                for (int64_t m = sc.j; m < m_tiles && ok; m += sc.G) {
                    for (int kb = 0; kb < k_blocks; ++kb) {
                        if (!mbar_wait_sleep(&tmem_empty[buf], aph ^ 1) || !mbar_wait_sleep(&full_bar[s], ph)) {
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t a_lo = ring_lo + s * (STAGE_BYTES >> 4);
                        const uint32_t b_lo = B_RES ? bres_lo + static_cast<uint32_t>(kb) * (kBBytes >> 4) : a_lo + (kABytes >> 4);
                        const uint64_t da = desc0 + a_lo;
                        const uint64_t db = desc0 + b_lo;
                        const uint32_t d_tmem = tmem_base + buf * kBN;
#pragma unroll
                        for (int k = 0; k < kBK / 32; ++k) mma_f8_ss(d_tmem, da + 2 * k, db + 2 * k, idesc, k > 0 ? 1u : 0u);
                        tc_commit(&empty_bar[s]);     // the stage may be refilled once these MMAs have read it
                        tc_commit(&tmem_full[buf]);   // the partial product of this K block is complete
                        if (++s == STAGES) {
                            s = 0;
                            ph ^= 1;
                        }
                        aph ^= buf;                   // the accumulator phase flips after buffer 1
                        buf ^= 1;
                    }
                }
            }
            if (!ok) {
                s_abort = 1;
                if (g.status != nullptr) atomicExch(g.status, 1);
            }
        }
    } else {
        // ---------------------------------------------------------------- promotion + epilogue
        const int et = threadIdx.x - 64;          // 0..511
        const int cq = et >> 7;                   // which 64-column quarter of the tile this thread serves
        const int quarter = warp & 3;             // TMEM lanes [32 * quarter, +32) are visible to this warp
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        // this thread's two 32-column ranges inside the 256-column accumulator
        const int col_a = MODE == kSwiGLU ? cq * 32 : cq * 64;
        const int col_b = MODE == kSwiGLU ? 128 + cq * 32 : cq * 64 + 32;
        const int nb_a = col_a >> 7;              // which of the tile's two 128-row weight blocks
        const int nb_b = col_b >> 7;
        uint32_t acc_it = 0;
        uint32_t tile_count = 0;
        bool ok = true;

        for (int n = sc.n_first; n < n_tiles && sc.active; n += sc.n_step) {
            const int n0 = n * kBN;
            // per-column-tile constants -> shared memory
            asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
            if (et < kBN) bias_s[et] = g.bias != nullptr ? g.bias[n0 + et] : 0.f;
            for (int i = et; i < 2 * k_blocks; i += kEpiThreads) {
                const int blk = i / k_blocks;
                const int kb = i - blk * k_blocks;
                sb_s[blk][kb] = g.sb[static_cast<int64_t>(n0 / 128 + blk) * k_blocks + kb];
            }
            asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");

            // activation scales are fetched two K blocks ahead of their use; the cursor walks the same
            // (row tile, K block) sequence as the main loop
            int64_t pf_m = sc.j;
            int pf_kb = 0;
            auto next_sa = [&]() -> float {
                float v = 0.f;
                if (pf_m < m_tiles) {
                    const int64_t r = pf_m * kBM + row_in_tile;
                    if (r < g.M) v = g.sa[r * k_blocks + pf_kb];
                    if (++pf_kb == k_blocks) {
                        pf_kb = 0;
                        pf_m += sc.G;
                    }
                }
                return v;
            };
            float sa_q0 = next_sa();
            float sa_q1 = next_sa();

            for (int64_t m = sc.j; m < m_tiles; m += sc.G, ++tile_count) {
                const int64_t row = m * kBM + row_in_tile;
                const bool row_ok = row < g.M;
                const int m0 = static_cast<int>(m) * kBM;
                if (MODE == kLinear && g.residual != nullptr && et == 0) {
                    // the staging tile is free once the previous tile's store has read it; the residual tile
                    // then lands in it while the K loop runs
                    bulk_wait_read<0>();
                    mbar_expect_tx(&res_full, P::kOutBytes);
#pragma unroll
                    for (int b = 0; b < P::kOutBoxes; ++b)
                        tma_load_2d(out_s + b * kOutBoxBytes, &tmap_r, 2 * n0 + b * 128, m0, &res_full);
                }

                // accumulators start from the bias: acc[0..15] <- columns col_a.., acc[16..31] <- col_b..
                float2 acc[32];
                if (g.bias == nullptr) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc[i] = make_float2(0.f, 0.f);
                } else {
                    const float4* ba = reinterpret_cast<const float4*>(bias_s + col_a);
                    const float4* bb = reinterpret_cast<const float4*>(bias_s + col_b);
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const float4 va = ba[i];
                        const float4 vb = bb[i];
                        acc[2 * i] = make_float2(va.x, va.y);
                        acc[2 * i + 1] = make_float2(va.z, va.w);
                        acc[16 + 2 * i] = make_float2(vb.x, vb.y);
                        acc[16 + 2 * i + 1] = make_float2(vb.z, vb.w);
                    }
                }

                for (int kb = 0; kb < k_blocks; ++kb, ++acc_it) {
                    const uint32_t buf = acc_it & 1;
                    const uint32_t aph = (acc_it >> 1) & 1;
                    const float sa = sa_q0;
                    sa_q0 = sa_q1;
                    sa_q1 = next_sa();
                    const float s_a = sa * sb_s[nb_a][kb];
                    const float s_b = sa * sb_s[nb_b][kb];
                    const float2 scale_a = make_float2(s_a, s_a);
                    const float2 scale_b = make_float2(s_b, s_b);
                    // A thread whose wait gives up does not leave the loop: it stops waiting (`ok` stays false) but
                    // walks the rest of the tile schedule, so it still meets every named barrier the other epilogue
                    // threads sit in.  Its results are garbage; the status word says so.
                    if (ok && !mbar_wait_sleep(&tmem_full[buf], aph)) ok = false;
                    tc_fence_after_sync();
                    const uint32_t t0 = tmem_base + buf * kBN + lane_addr;
                    // 16 columns at a time: the accumulators already take 64 of the 96 registers a thread may use
                    uint32_t r[16];
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        tmem_ld_x16(t0 + (c < 2 ? col_a + 16 * c : col_b + 16 * (c - 2)), r);
                        tc_wait_ld();
                        const float2 sc2 = c < 2 ? scale_a : scale_b;
#pragma unroll
                        for (int i = 0; i < 8; ++i)
                            acc[8 * c + i] = __ffma2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), sc2, acc[8 * c + i]);
                    }
                    tc_fence_before_sync();
                    mbar_arrive(&tmem_empty[buf]);
                }
                // -------------------------------------------------------- tile epilogue
                // Staging address of this thread's 16-byte piece j of its row (128-byte swizzle: piece ^ row % 8)
                const int swz = row_in_tile & 7;
                if (MODE == kSwiGLU || MODE == kSiLU) {
                    // kSwiGLU: acc[0..15] = gate, acc[16..31] = value of hidden columns h0 + cq * 32 + (0..31);
                    //          the 128-column quantisation block of the row is shared by the four column quarters.
                    // kSiLU:   64 hidden columns n0 + cq * 64 + (0..63); the block is shared by two quarters.
                    constexpr int NV = MODE == kSwiGLU ? 16 : 32;  // float2 values this thread produces
                    float amax = 0.f;
#pragma unroll
                    for (int i = 0; i < NV; ++i) {
                        float2 h;
                        h = make_float2(silu(acc[i].x), silu(acc[i].y));
                        if (MODE == kSwiGLU) h = __fmul2_rn(h, acc[16 + i]);
                        acc[i] = h;
                        amax = fmaxf(amax, fmaxf(fabsf(h.x), fabsf(h.y)));
                    }
                    float (*xchg)[kBM] = amax_xchg[tile_count & 1];  // alternate buffers: no third barrier per tile
                    xchg[cq][row_in_tile] = amax;
                    if (et == 0) bulk_wait_read<0>();       // the previous tile's store has read the staging tile
                    asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
                    if (MODE == kSwiGLU) {
                        amax = fmaxf(fmaxf(xchg[0][row_in_tile], xchg[1][row_in_tile]),
                                     fmaxf(xchg[2][row_in_tile], xchg[3][row_in_tile]));
                    } else {
                        amax = fmaxf(amax, xchg[cq ^ 1][row_in_tile]);
                    }
                    const float scale = amax > 0.f ? amax / 448.0f : 1.0f;
                    const float inv1 = 1.0f / scale;
                    const float2 inv = make_float2(inv1, inv1);
                    // kSwiGLU: one box, pieces cq * 2 + {0, 1}; kSiLU: box cq / 2, pieces (cq % 2) * 4 + {0..3}
                    uint8_t* box_row = out_s + (MODE == kSiLU ? (cq >> 1) * kOutBoxBytes : 0) + row_in_tile * 128;
                    const int piece0 = MODE == kSwiGLU ? cq * 2 : (cq & 1) * 4;
#pragma unroll
                    for (int c = 0; c < NV / 8; ++c) {
                        uint32_t w[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const float2 lo = __fmul2_rn(acc[8 * c + 2 * e], inv);
                            const float2 hi = __fmul2_rn(acc[8 * c + 2 * e + 1], inv);
                            w[e] = static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(lo, __NV_SATFINITE, __NV_E4M3)) |
                                   (static_cast<uint32_t>(__nv_cvt_float2_to_fp8x2(hi, __NV_SATFINITE, __NV_E4M3)) << 16);
                        }
                        *reinterpret_cast<uint4*>(box_row + (((piece0 + c) ^ swz) << 4)) = make_uint4(w[0], w[1], w[2], w[3]);
                    }
                    if (row_ok) {
                        if (MODE == kSwiGLU) {
                            if (cq == 0) g.out_scale[row * (g.N / 256) + n0 / kBN] = scale;
                        } else if ((cq & 1) == 0) {
                            g.out_scale[row * (g.N / 128) + (n0 + cq * 64) / 128] = scale;
                        }
                    }
                } else {
                    // 64 bf16 columns = one 128-byte box row per thread: box cq, pieces 0..7
                    uint8_t* box_row = out_s + cq * kOutBoxBytes + row_in_tile * 128;
                    const bool has_res = g.residual != nullptr;
                    if (et == 0) bulk_wait_read<0>();
                    asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
                    if (has_res && ok && !mbar_wait_sleep(&res_full, tile_count & 1)) ok = false;   // keep going, see above
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        uint4* slot = reinterpret_cast<uint4*>(box_row + ((c ^ swz) << 4));
                        float2 v[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[e] = acc[4 * c + e];
                        if (has_res) {
                            float2 rr[4];
                            Vec16<__nv_bfloat16>::unpack2(*slot, rr);
#pragma unroll
                            for (int e = 0; e < 4; ++e) v[e] = __fadd2_rn(v[e], rr[e]);
                        }
                        *slot = Vec16<__nv_bfloat16>::pack2(v);
                    }
                }
                // staging tile complete -> one thread hands it to TMA (rows past M are clipped by the tensor map)
                fence_proxy_async_smem();
                asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
                if (et == 0) {
                    const int x0 = MODE == kSwiGLU ? (n0 / kBN) * 128 : (MODE == kSiLU ? n0 : 2 * n0);
#pragma unroll
                    for (int b = 0; b < P::kOutBoxes; ++b) tma_store_2d(&tmap_o, out_s + b * kOutBoxBytes, x0 + b * 128, m0);
                    bulk_commit();
                }
            }
        }
        if (et == 0) bulk_wait<0>();   // the last store must have left shared memory before the CTA ends
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
// activation quantisation: bf16 [M, K] -> e4m3 [M, K] + fp32 scales [M, K / 128]
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
quant_act_kernel(const uint4* __restrict__ x, uint2* __restrict__ q, float* __restrict__ scales, int64_t n_blocks) {
    // 16 lanes x 8 values = one 1 x 128 block
    const int64_t gthread = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    const int64_t block = gthread >> 4;
    const int sub = threadIdx.x & 15;
    const bool ok = block < n_blocks;
    float f[8];
    if (ok) {
        Vec16<__nv_bfloat16>::unpack(x[block * 16 + sub], f);
    } else {
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = 0.f;
    }
    float amax = 0.f;
#pragma unroll
    for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(f[e]));
#pragma unroll
    for (int o = 8; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float scale = amax > 0.f ? amax / 448.0f : 1.0f;
    const float inv = 1.0f / scale;
    if (ok) {
        uint2 w;
        w.x = pack_e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
        w.y = pack_e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
        q[block * 16 + sub] = w;
        if (sub == 0) scales[block] = scale;
    }
}

// ------------------------------------------------------------------------------------------------
// host side
// ------------------------------------------------------------------------------------------------
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

// [rows, k_bytes] row-major bytes, tiles of box_rows x 128 bytes, 128-byte swizzle, zero fill outside
bool make_tmap_bytes(CUtensorMap* map, const void* base, uint64_t k_bytes, uint64_t rows, uint64_t pitch_bytes,
                     uint32_t box_rows) {
    PFN_cuTensorMapEncodeTiled_v12000 fn = encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {k_bytes, rows};
    const cuuint64_t strides[1] = {pitch_bytes};
    const cuuint32_t box[2] = {static_cast<cuuint32_t>(kBK), box_rows};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int MODE, bool B_RES>
int launch_gemm_impl(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, const CUtensorMap& tr,
                     const GemmArgs& g, cudaStream_t stream) {
    using P = Plan<MODE, B_RES>;
    const DeviceInfo& dev = device_info();
    const size_t smem = P::tiles_bytes(g.K / kBK) + 1024;
    static bool attr_set[64] = {};
    if (!attr_set[dev.index]) {
        cudaFuncSetAttribute(ffn_gemm_kernel<MODE, B_RES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(P::tiles_bytes(4) + 1024));
        attr_set[dev.index] = true;
    }
    const int64_t m_tiles = (g.M + kBM - 1) / kBM;
    const int n_tiles = g.N / kBN;
    int64_t grid = dev.sm_count;
    if (n_tiles <= grid) {  // no more row walkers per column tile than there are row tiles
        int64_t walkers = grid / n_tiles;
        if (walkers > m_tiles) walkers = m_tiles;
        grid = walkers * n_tiles;
    }
    ffn_gemm_kernel<MODE, B_RES><<<static_cast<unsigned>(grid), kThreads, smem, stream>>>(ta, tb, to, tr, g);
    count_launch();
    return launch_status();
}

template <int MODE>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, const CUtensorMap& tr,
                const GemmArgs& g, cudaStream_t stream) {
    // the resident weight tile pays off for the short K of the up projection; the linear mode needs the room
    // for its 64 KB staging tile instead
    if (MODE != kLinear && g.K <= 4 * kBK) return launch_gemm_impl<MODE, true>(ta, tb, to, tr, g, stream);
    return launch_gemm_impl<MODE, false>(ta, tb, to, tr, g, stream);
}

// ------------------------------------------------------------------------------------------------
// Fixed scratch for callers that must not allocate
// ------------------------------------------------------------------------------------------------
// The whole FFN (quantise -> GEMM 1 -> GEMM 2) needs the quantised input, the e4m3 hidden activation
// and their scale vectors between its three kernels.  tb200_ffn_fp8_fwd_static keeps them in this
// array, which lives in the library's device image: every GPU that loads the library holds these
// bytes until the process exits, and every call on that GPU shares them.
constexpr size_t kStaticScratchBytes = size_t(64) << 20;
constexpr size_t kStaticStatusBytes = 256;   // the array's first bytes: the status word the two GEMMs raise
static __device__ __align__(256) uint8_t g_ffn_scratch[kStaticScratchBytes];

// In host code `g_ffn_scratch` is only a handle for the runtime, not a device address; the address
// a kernel can use comes from cudaGetSymbolAddress, asked once per device with that device current.
int static_scratch_base(uint8_t** base) {
    static std::mutex lock;
    static uint8_t* cached[64] = {};
    const DeviceInfo& dev = device_info();
    if (!dev.valid) return TB200_ERR_DEVICE;
    std::lock_guard<std::mutex> guard(lock);
    if (cached[dev.index] == nullptr) {
        void* ptr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&ptr, g_ffn_scratch);
        if (e != cudaSuccess) return static_cast<int>(e);
        cached[dev.index] = static_cast<uint8_t*>(ptr);
    }
    *base = cached[dev.index];
    return TB200_OK;
}

inline size_t round256(size_t v) { return (v + 255) & ~size_t(255); }

}  // namespace
}  // namespace tb200

extern "C" int tb200_quant_act_1x128(const void* x_bf16, void* x_fp8, float* scales, int64_t M, int32_t K,
                                     void* stream) {
    using namespace tb200;
    if (M < 0 || K < 128 || K % 128 != 0) return TB200_ERR_SHAPE;
    if (M == 0) return TB200_OK;
    if (x_bf16 == nullptr || x_fp8 == nullptr || scales == nullptr) return TB200_ERR_NULL;
    if (!aligned16(x_bf16) || !aligned16(x_fp8)) return TB200_ERR_ALIGN;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    const int64_t n_blocks = M * (K / 128);
    const int64_t grid = (n_blocks * 16 + 255) / 256;
    if (grid > 0x7FFFFFFFll) return TB200_ERR_SHAPE;
    quant_act_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(x_bf16), static_cast<uint2*>(x_fp8), scales, n_blocks);
    count_launch();
    return launch_status();
}

extern "C" int tb200_fp8_gemm(const void* a_fp8, const float* a_scales, const void* b_fp8, const float* b_scales,
                              const float* bias, const void* residual, void* out, float* out_scales, int64_t M,
                              int32_t N, int32_t K, int32_t mode, int32_t* status_word, void* stream) {
    using namespace tb200;
    if (M < 0 || N < 256 || N % 256 != 0 || K < 128 || K % 128 != 0 || K > 8192) return TB200_ERR_SHAPE;
    if (mode < 0 || mode > 2) return TB200_ERR_UNSUPPORTED;
    if (M == 0) return TB200_OK;
    if (a_fp8 == nullptr || a_scales == nullptr || b_fp8 == nullptr || b_scales == nullptr || out == nullptr)
        return TB200_ERR_NULL;
    if (mode != kLinear && out_scales == nullptr) return TB200_ERR_NULL;
    if (mode != kLinear && residual != nullptr) return TB200_ERR_UNSUPPORTED;
    if (!aligned16(a_fp8) || !aligned16(b_fp8) || !aligned16(out) || (residual != nullptr && !aligned16(residual)))
        return TB200_ERR_ALIGN;
    if (M > 0x7FFFFF00ll) return TB200_ERR_SHAPE;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    CUtensorMap ta, tb;
    if (!make_tmap_bytes(&ta, a_fp8, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(K), kBM) ||
        !make_tmap_bytes(&tb, b_fp8, static_cast<uint64_t>(K), static_cast<uint64_t>(N), static_cast<uint64_t>(K), kBN))
        return TB200_ERR_DRIVER;
    // output (and residual) as byte matrices in boxes of 128 rows x 128 bytes
    const uint64_t out_row_bytes = mode == kSwiGLU ? static_cast<uint64_t>(N) / 2 : (mode == kSiLU ? static_cast<uint64_t>(N) : 2ull * N);
    CUtensorMap to, tr;
    if (!make_tmap_bytes(&to, out, out_row_bytes, static_cast<uint64_t>(M), out_row_bytes, kBM)) return TB200_ERR_DRIVER;
    if (!make_tmap_bytes(&tr, residual != nullptr ? residual : out, out_row_bytes, static_cast<uint64_t>(M), out_row_bytes, kBM))
        return TB200_ERR_DRIVER;
    GemmArgs g{};
    g.sa = a_scales;
    g.sb = b_scales;
    g.bias = bias;
    g.residual = static_cast<const __nv_bfloat16*>(residual);
    g.out = out;
    g.out_scale = out_scales;
    g.status = status_word;
    g.M = M;
    g.N = N;
    g.K = K;
    g.out_ld = mode == kSwiGLU ? N / 2 : N;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (mode == kSwiGLU) return launch_gemm<kSwiGLU>(ta, tb, to, tr, g, s);
    if (mode == kSiLU) return launch_gemm<kSiLU>(ta, tb, to, tr, g, s);
    return launch_gemm<kLinear>(ta, tb, to, tr, g, s);
}

extern "C" int64_t tb200_ffn_fp8_static_scratch_bytes(void) { return static_cast<int64_t>(tb200::kStaticScratchBytes); }

extern "C" int tb200_ffn_fp8_fwd_static(const void* x_bf16, const void* w_up_fp8, const float* w_up_scales,
                                        const float* b_up, const void* w_down_fp8, const float* w_down_scales,
                                        const float* b_down, const void* residual, void* y_bf16, int64_t M,
                                        int32_t d_in, int32_t hidden, int32_t d_out, int32_t gated, void* stream) {
    using namespace tb200;
    // Every check that one of the three sub-calls would make comes first, so that a negative return
    // really means "nothing was launched".
    if (M < 0 || d_in < 128 || d_in % 128 != 0 || d_in > 8192 || hidden < 256 || hidden % 256 != 0 || hidden > 8192 ||
        d_out < 256 || d_out % 256 != 0)
        return TB200_ERR_SHAPE;
    if (M == 0) return TB200_OK;
    // the array bounds the rows long before the products below could wrap, or the GEMMs' own row limit is reached
    if (M > static_cast<int64_t>(kStaticScratchBytes)) return TB200_ERR_SCRATCH;
    if (x_bf16 == nullptr || w_up_fp8 == nullptr || w_up_scales == nullptr || w_down_fp8 == nullptr ||
        w_down_scales == nullptr || y_bf16 == nullptr)
        return TB200_ERR_NULL;
    if (!aligned16(x_bf16) || !aligned16(w_up_fp8) || !aligned16(w_down_fp8) || !aligned16(y_bf16) ||
        (residual != nullptr && !aligned16(residual)))
        return TB200_ERR_ALIGN;
    // carve the fixed array: [status word | x e4m3 | x scales | hidden e4m3 | hidden scales], each part 256-byte aligned
    const size_t um = static_cast<size_t>(M);
    const size_t xq_bytes = round256(um * d_in);
    const size_t sx_bytes = round256(um * (d_in / 128) * sizeof(float));
    const size_t h_bytes = round256(um * hidden);
    const size_t sh_bytes = round256(um * (hidden / 128) * sizeof(float));
    if (kStaticStatusBytes + xq_bytes + sx_bytes + h_bytes + sh_bytes > kStaticScratchBytes) return TB200_ERR_SCRATCH;
    uint8_t* base = nullptr;
    const int rc = static_scratch_base(&base);
    if (rc != TB200_OK) return rc;
    int32_t* status = reinterpret_cast<int32_t*>(base);
    uint8_t* xq = base + kStaticStatusBytes;
    float* sx = reinterpret_cast<float*>(xq + xq_bytes);
    uint8_t* h = xq + xq_bytes + sx_bytes;
    float* sh = reinterpret_cast<float*>(h + h_bytes);
    // The status word is the one part of the array that must start at zero: the kernels only ever raise it.
    // The data parts need no clearing, the three kernels overwrite every byte they later read (rows [0, M)).
    const cudaError_t e = cudaMemsetAsync(status, 0, sizeof(int32_t), static_cast<cudaStream_t>(stream));
    if (e != cudaSuccess) return static_cast<int>(e);
    int code = tb200_quant_act_1x128(x_bf16, xq, sx, M, d_in, stream);
    if (code != TB200_OK) return code;
    code = tb200_fp8_gemm(xq, sx, w_up_fp8, w_up_scales, b_up, nullptr, h, sh, M, gated ? 2 * hidden : hidden, d_in,
                          gated ? 0 : 1, status, stream);
    if (code != TB200_OK) return code;
    return tb200_fp8_gemm(h, sh, w_down_fp8, w_down_scales, b_down, residual, y_bf16, nullptr, M, d_out, hidden, 2,
                          status, stream);
}

extern "C" int tb200_ffn_fp8_static_status(void* stream, int32_t* value) {
    using namespace tb200;
    if (value == nullptr) return TB200_ERR_NULL;
    uint8_t* base = nullptr;
    const int rc = static_scratch_base(&base);
    if (rc != TB200_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    cudaError_t e = cudaMemcpyAsync(value, base, sizeof(int32_t), cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    return e == cudaSuccess ? TB200_OK : static_cast<int>(e);
}
