// FP8 (e4m3) FFN with power-of-two block scales applied by the tensor cores themselves (sm_100a
// `tcgen05.mma.kind::mxf8f6f4.block_scale`): activation quantisation and the two GEMMs, with bias, SiLU / SiLU-gating
// and the re-quantisation of the hidden activation in the GEMM epilogues.
//
// Same block structure as the amax/448 path of ffn_fp8.cu — one scale per 1 x 128 block of an activation row, one per
// 128 x 128 block of a weight, both derived from the block's amax — but the scale is rounded UP to a power of two
// (UE8M0: one exponent byte, value 2^(byte - 127)), the format the hardware multiplies in: every 32-wide K slice of
// an MMA takes one scale per row of A and one per row of B from tensor memory.  A 1 x 128 scale is simply repeated
// for its four slices.  The whole K range of an output tile therefore accumulates in ONE tensor-memory accumulator and
// the epilogue reads it once per tile, instead of promoting a partial product per K block on the CUDA cores (which is
// what bounds the amax/448 kernel).  Rounding the scale up costs at most one binade of e4m3's dynamic range (values
// use [224, 448] -> (112, 448] of the code range); the mantissa, hence the rounding error, is unchanged.
//
// Scale factors travel in the layout the copy into tensor memory wants, one 512-byte atom per (128 rows, 128-wide K
// block): byte (r % 32) * 16 + (r / 32) * 4 + s holds the scale of row r, slice s.  Activations:
// [ceil(M / 128), K / 128, 512]; weights: [N / 128, K / 128, 512].
//
// Roles in a CTA of 576 threads (persistent, one CTA per SM, static round-robin over output tiles):
//   warp 0       producer: ring of {A 128 x 128 B, B 256 x 128 B} tiles by TMA (128-byte swizzle) plus their scale atoms
//                by bulk copies, all counted on the stage's barrier
//   warp 1       MMA issuer (one elected lane), owner of the TMEM allocation: per K block it copies the scale atoms
//                into TMEM (`tcgen05.cp`, alternating between two slots) and issues four 128 x 256 x 32 MMAs
//   warps 2..17  epilogue: a thread owns one output row and 64 of the 256 columns; it drains its part of the
//                accumulator into registers and releases the accumulator at once, so the MMAs of the next tile run
//                under the epilogue's arithmetic and stores.  The four warps of a TMEM lane quarter work as a group
//                with their own named barrier, staging rows and TMA stores: nothing inside a tile waits for all
//                sixteen warps
// Every wait on an mbarrier is bounded; a wait that gives up raises the status word and all roles drain out through
// the same final barrier, where the TMEM allocation is released.
#include <cstdlib>

#include <cuda_fp8.h>
#include <cudaTypedefs.h>

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
constexpr uint32_t kABytes = kBM * kBK;      // 16 KB
constexpr uint32_t kBBytes = kBN * kBK;      // 32 KB
constexpr uint32_t kSfAtom = 512;            // scale factors of 128 rows x one K block
constexpr uint32_t kSfaBytes = kSfAtom;      // A: 128 rows
constexpr uint32_t kSfbBytes = 2 * kSfAtom;  // B: 256 rows
constexpr uint32_t kTmemCols = 512;          // accumulator 256 + two scale-factor slots of 12 columns (allocation: power of two)
constexpr uint32_t kTmemSf = 256;            // first scale-factor column
constexpr uint32_t kSfSlotCols = 12;         // a per-K-block slot: 4 columns for A, 8 for B
constexpr uint32_t kTmemSfbRes = kTmemSf + 2 * kSfSlotCols;   // resident weight scales (B_RES): 8 columns per K block

enum Mode : int {
    kSwiGLU = 0,  // columns = [128 gate | 128 up] of one hidden block -> e4m3 hidden + scale atoms
    kSiLU = 1,    // hidden = silu(acc + bias)                          -> e4m3 hidden + scale atoms
    kLinear = 2,  // y = acc + bias (+ residual)                        -> bf16
};

struct GemmArgs {
    const uint8_t* sfa;  // [m_tiles, K / 128, 512] activation scale atoms
    const uint8_t* sfb;  // [N / 128, K / 128, 512] weight scale atoms
    const float* bias;   // [N] fp32 or nullptr (for kSwiGLU in the tile's interleaved column order)
    const __nv_bfloat16* residual;  // [M, N] or nullptr (kLinear only)
    void* out;           // kLinear: bf16 [M, N]; else e4m3 [M, N_hidden]
    uint8_t* out_sf;     // [m_tiles, N_hidden / 128, 512] scale atoms of the hidden activation (quantising modes)
    int32_t* status;     // device word: set to 1 when a wait gave up (may be nullptr)
    int64_t M;
    int32_t N;           // GEMM columns (kSwiGLU: 2 * hidden)
    int32_t K;
};

__device__ __forceinline__ float silu(float x) {
    const float h = 0.5f * x;
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(h));
    return fmaf(h, t, h);
}

// Smallest power of two s with amax / s <= 448, as its UE8M0 byte (s = 2^(byte - 127)), and 1 / s.
__device__ __forceinline__ uint32_t pow2_scale(float amax, float* inv) {
    int e = 0;
    if (amax > 0.f) {
        const uint32_t bits = __float_as_uint(amax * (1.0f / 448.0f));
        e = static_cast<int>((bits >> 23) & 0xFF) - 127 + ((bits & 0x7FFFFFu) != 0u ? 1 : 0);
        e = max(-126, min(e, 126));
    }
    *inv = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);
    return static_cast<uint32_t>(e + 127);
}

__device__ __forceinline__ uint32_t pack_e4m3x4(float a, float b, float c, float d) {
    const __nv_fp8x2_storage_t lo = __nv_cvt_float2_to_fp8x2(make_float2(a, b), __NV_SATFINITE, __NV_E4M3);
    const __nv_fp8x2_storage_t hi = __nv_cvt_float2_to_fp8x2(make_float2(c, d), __NV_SATFINITE, __NV_E4M3);
    return static_cast<uint32_t>(lo) | (static_cast<uint32_t>(hi) << 16);
}

// byte offset of row r's four slice bytes inside a scale atom
__host__ __device__ __forceinline__ uint32_t sf_row_offset(int r) { return static_cast<uint32_t>((r & 31) * 16 + (r >> 5) * 4); }

// Work distribution as in the amax/448 kernel: a CTA keeps ONE column tile for its whole life and walks down the row
// tiles; the CTAs that share a row tile read it at about the same time, so activations come from HBM once.
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
        sc.n_step = 0x40000000;
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

constexpr int kMaxStages = 7;
constexpr uint32_t kOutBoxBytes = kBM * 128;   // one staging box: 128 rows x 128 bytes, 128-byte swizzle

// Shared-memory plan.  With B_RES (K <= 512) the weight tile and its scale atoms stay resident and only the activation
// tiles stream through the ring; a ring stage is padded to a multiple of 1 KB (the swizzled tiles need that alignment).
template <int MODE, bool B_RES>
struct Plan {
    static constexpr int kOutBoxes = MODE == kSwiGLU ? 1 : (MODE == kSiLU ? 2 : 4);
    static constexpr uint32_t kOutBytes = kOutBoxes * kOutBoxBytes;
    static constexpr int kStagesN = B_RES ? (MODE == kSiLU ? 3 : 4) : 3;     // the SiLU mode stages two output boxes
    static constexpr uint32_t kStageBytesN = B_RES ? kABytes + 1024 : kABytes + kBBytes + 2048;
    static constexpr uint32_t kStageTx = B_RES ? kABytes + kSfaBytes : kABytes + kBBytes + kSfaBytes + kSfbBytes;
    static constexpr size_t tiles_bytes(int k_blocks) {
        return (B_RES ? static_cast<size_t>(k_blocks) * (kBBytes + kSfbBytes) : 0) + static_cast<size_t>(kStagesN) * kStageBytesN +
               kOutBytes;
    }
};

template <int MODE, bool B_RES>
__global__ void __launch_bounds__(kThreads, 1)
mx_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ CUtensorMap tmap_o, const __grid_constant__ CUtensorMap tmap_r, const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[kMaxStages];
    __shared__ uint64_t empty_bar[kMaxStages];
    __shared__ uint64_t b_full;
    __shared__ uint64_t res_full[4];   // one per TMEM lane quarter: the residual rows of that quarter have landed
    __shared__ uint64_t tmem_full;
    __shared__ uint64_t tmem_empty;
    __shared__ uint32_t tmem_base_slot;
    __shared__ __align__(16) float bias_s[kBN];
    __shared__ float amax_xchg[2][4][kBM];
    __shared__ int s_abort;

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const int64_t m_tiles = (g.M + kBM - 1) / kBM;
    const int n_tiles = g.N / kBN;
    const int k_blocks = g.K / kBK;
    using P = Plan<MODE, B_RES>;
    constexpr int STAGES = P::kStagesN;
    constexpr uint32_t STAGE_BYTES = P::kStageBytesN;
    // resident weights: [k_blocks][32 KB] tiles, then [k_blocks][1 KB] scale atoms; then the ring; then the staging tile
    uint8_t* b_res = smem;
    uint8_t* sfb_res = smem + static_cast<size_t>(k_blocks) * kBBytes;
    uint8_t* ring = B_RES ? smem + static_cast<size_t>(k_blocks) * (kBBytes + kSfbBytes) : smem;
    uint8_t* out_s = ring + static_cast<size_t>(STAGES) * STAGE_BYTES;
    // inside a ring stage: A tile, (B tile,) scale atoms of A (and of B)
    constexpr uint32_t kSfaInStage = B_RES ? kABytes : kABytes + kBBytes;
    constexpr uint32_t kSfbInStage = kSfaInStage + kSfaBytes;
    const Schedule sc = make_schedule(n_tiles);

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&b_full, 1);
        for (int q = 0; q < 4; ++q) mbar_init(&res_full[q], 1);
        mbar_init(&tmem_full, 1);
        mbar_init(&tmem_empty, kEpiThreads);
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
        // ---------------------------------------------------------------- producer
        if (lane == 0 && sc.active) {
            tma_prefetch_desc(&tmap_a);
            tma_prefetch_desc(&tmap_b);
            uint32_t it = 0;
            bool ok = true;
            for (int n = sc.n_first; n < n_tiles && ok; n += sc.n_step) {
                const int n0 = n * kBN;
                const uint8_t* sfb_n = g.sfb + static_cast<int64_t>(n0 / 128) * k_blocks * kSfAtom;   // two weight blocks: n0/128, +1
                if (B_RES) {
                    if (it > 0) {  // the previous column tile's MMAs must have finished reading the resident tile
                        const uint32_t last = it - 1;
                        if (!mbar_wait_sleep(&empty_bar[last % STAGES], (last / STAGES) & 1)) { ok = false; break; }
                    }
                    mbar_expect_tx(&b_full, static_cast<uint32_t>(k_blocks) * (kBBytes + kSfbBytes));
                    for (int kb = 0; kb < k_blocks; ++kb) {
                        tma_load_2d(b_res + static_cast<size_t>(kb) * kBBytes, &tmap_b, kb * kBK, n0, &b_full);
                        bulk_load(sfb_res + kb * kSfbBytes, sfb_n + static_cast<int64_t>(kb) * kSfAtom, kSfAtom, &b_full);
                        bulk_load(sfb_res + kb * kSfbBytes + kSfAtom, sfb_n + (static_cast<int64_t>(k_blocks) + kb) * kSfAtom, kSfAtom,
                                  &b_full);
                    }
                }
                for (int64_t m = sc.j; m < m_tiles && ok; m += sc.G) {
                    const int m0 = static_cast<int>(m) * kBM;
                    const uint8_t* sfa_m = g.sfa + m * k_blocks * kSfAtom;
                    for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                        const uint32_t s = it % STAGES;
                        const uint32_t ph = (it / STAGES) & 1;
                        if (!mbar_wait_sleep(&empty_bar[s], ph ^ 1) || *reinterpret_cast<volatile int*>(&s_abort)) {
                            ok = false;
                            break;
                        }
                        uint8_t* stage = ring + static_cast<size_t>(s) * STAGE_BYTES;
                        mbar_expect_tx(&full_bar[s], P::kStageTx);
                        tma_load_2d(stage, &tmap_a, kb * kBK, m0, &full_bar[s]);
                        bulk_load(stage + kSfaInStage, sfa_m + static_cast<int64_t>(kb) * kSfAtom, kSfAtom, &full_bar[s]);
                        if (!B_RES) {
                            tma_load_2d(stage + kABytes, &tmap_b, kb * kBK, n0, &full_bar[s]);
                            bulk_load(stage + kSfbInStage, sfb_n + static_cast<int64_t>(kb) * kSfAtom, kSfAtom, &full_bar[s]);
                            bulk_load(stage + kSfbInStage + kSfAtom, sfb_n + (static_cast<int64_t>(k_blocks) + kb) * kSfAtom, kSfAtom,
                                      &full_bar[s]);
                        }
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
            const uint64_t desc0 = umma_desc_sw128(0, 1024, 16);
            const uint64_t sf_desc0 = umma_desc_noswizzle(0, 128, 0);      // 32 rows x 16 bytes: four 8-row groups 128 B apart
            const uint32_t ring_lo = (smem_u32(ring) & 0x3FFFFu) >> 4;
            const uint32_t bres_lo = B_RES ? (smem_u32(b_res) & 0x3FFFFu) >> 4 : 0u;
            const uint32_t sfbres_lo = B_RES ? (smem_u32(sfb_res) & 0x3FFFFu) >> 4 : 0u;
            uint32_t s = 0, ph = 0, b_phase = 0, tile = 0, it = 0;
            bool ok = true;
            for (int n = sc.n_first; n < n_tiles && ok; n += sc.n_step) {
                if (B_RES) {
                    if (!mbar_wait_sleep(&b_full, b_phase)) { ok = false; break; }
                    b_phase ^= 1;
                    tc_fence_after_sync();
                    // the resident weight tile's scale factors go into tensor memory once per column tile
                    // (ordered behind the MMAs of the previous column tile, which read the same columns)
                    for (int kb = 0; kb < k_blocks; ++kb) {
                        const uint32_t src = sfbres_lo + static_cast<uint32_t>(kb) * (kSfbBytes >> 4);
                        tc_cp_32x128b_warpx4(tmem_base + kTmemSfbRes + kb * 8, sf_desc0 + src);
                        tc_cp_32x128b_warpx4(tmem_base + kTmemSfbRes + kb * 8 + 4, sf_desc0 + src + (kSfAtom >> 4));
                    }
                }
                for (int64_t m = sc.j; m < m_tiles && ok; m += sc.G, ++tile) {
                    // the epilogue has read the previous tile out of the accumulator
                    if (!mbar_wait_sleep(&tmem_empty, (tile & 1) ^ 1)) { ok = false; break; }
                    tc_fence_after_sync();
                    for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                        if (!mbar_wait_sleep(&full_bar[s], ph)) { ok = false; break; }
                        tc_fence_after_sync();
                        const uint32_t a_lo = ring_lo + s * (STAGE_BYTES >> 4);
                        const uint32_t b_lo = B_RES ? bres_lo + static_cast<uint32_t>(kb) * (kBBytes >> 4) : a_lo + (kABytes >> 4);
                        const uint32_t sfa_lo = a_lo + (kSfaInStage >> 4);
                        const uint32_t sfb_lo = B_RES ? sfbres_lo + static_cast<uint32_t>(kb) * (kSfbBytes >> 4) : a_lo + (kSfbInStage >> 4);
                        // scale factors of this K block -> TMEM slot (it & 1): 4 columns for A, 8 for B
                        const uint32_t t_sfa = tmem_base + kTmemSf + (it & 1) * kSfSlotCols;
                        const uint32_t t_sfb = B_RES ? tmem_base + kTmemSfbRes + kb * 8 : t_sfa + 4;
                        tc_cp_32x128b_warpx4(t_sfa, sf_desc0 + sfa_lo);
                        if (!B_RES) {
                            tc_cp_32x128b_warpx4(t_sfb, sf_desc0 + sfb_lo);
                            tc_cp_32x128b_warpx4(t_sfb + 4, sf_desc0 + sfb_lo + (kSfAtom >> 4));
                        }
                        const uint64_t da = desc0 + a_lo;
                        const uint64_t db = desc0 + b_lo;
#pragma unroll
                        for (int k = 0; k < kBK / 32; ++k)
                            mma_mxf8_ss(tmem_base, da + 2 * k, db + 2 * k, umma_idesc_mx(kBM, kBN, k, k), (kb > 0 || k > 0) ? 1u : 0u,
                                        t_sfa, t_sfb);
                        tc_commit(&empty_bar[s]);     // the stage may be refilled once these MMAs have read it
                        if (++s == STAGES) {
                            s = 0;
                            ph ^= 1;
                        }
                    }
                    if (ok) tc_commit(&tmem_full);    // the tile's accumulator is complete
                }
            }
            if (!ok) {
                s_abort = 1;
                if (g.status != nullptr) atomicExch(g.status, 1);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue
        // The four warps that share a TMEM lane quarter (32 output rows, one 64-column quarter each) form a group of their
        // own: they exchange the row amax, fill their 32 rows of the staging boxes and send them off with their own TMA
        // stores, synchronised by a named barrier of 128 threads.  No barrier spans all sixteen warps inside a tile, so
        // the groups drift apart and one group's conversions overlap another's special-function work.
        const int et = threadIdx.x - 64;          // 0..511
        const int cq = et >> 7;                   // which 64-column quarter of the tile this thread serves
        const int quarter = warp & 3;             // TMEM lanes [32 * quarter, +32) are visible to this warp
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        const int col_a = MODE == kSwiGLU ? cq * 32 : cq * 64;
        const int col_b = MODE == kSwiGLU ? 128 + cq * 32 : cq * 64 + 32;
        const bool leader = cq == 0 && lane == 0; // issues the group's TMA loads and stores
        const uint32_t group_bar = 2 + quarter;
        uint8_t* out_q = out_s + quarter * 4096;  // this group's 32 rows inside every 16 KB staging box
        uint32_t tile_count = 0;
        bool ok = true;

        for (int n = sc.n_first; n < n_tiles && sc.active; n += sc.n_step) {
            const int n0 = n * kBN;
            asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
            if (et < kBN) bias_s[et] = g.bias != nullptr ? g.bias[n0 + et] : 0.f;
            asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");

            for (int64_t m = sc.j; m < m_tiles; m += sc.G, ++tile_count) {
                const int64_t row = m * kBM + row_in_tile;
                const bool row_ok = row < g.M;
                const int m0 = static_cast<int>(m) * kBM;
                if (MODE == kLinear && g.residual != nullptr && leader) {
                    // the group's staging rows are free once its previous stores have read them; the residual rows
                    // then land there while the K loop runs
                    bulk_wait_read<0>();
                    mbar_expect_tx(&res_full[quarter], P::kOutBoxes * 4096u);
#pragma unroll
                    for (int b = 0; b < P::kOutBoxes; ++b)
                        tma_load_2d(out_q + b * kOutBoxBytes, &tmap_r, 2 * n0 + b * 128, m0 + quarter * 32, &res_full[quarter]);
                }
                // A thread whose wait gives up keeps walking the schedule (it still meets every named barrier); its
                // results are garbage and the status word says so.
                if (ok && !mbar_wait_sleep(&tmem_full, tile_count & 1)) ok = false;
                tc_fence_after_sync();
                // drain this thread's 64 columns into registers (bias added on the way), then release the accumulator
                float2 acc[32];
                const uint32_t t0 = tmem_base + lane_addr;
                {
                    uint32_t r0[16], r1[16], r2[16], r3[16];     // four loads in flight under one wait
                    tmem_ld_x16(t0 + col_a, r0);
                    tmem_ld_x16(t0 + col_a + 16, r1);
                    tmem_ld_x16(t0 + col_b, r2);
                    tmem_ld_x16(t0 + col_b + 16, r3);
                    tc_wait_ld(r0);
                    tc_wait_ld(r1);
                    tc_wait_ld(r2);
                    tc_wait_ld(r3);
                    const float4* ba = reinterpret_cast<const float4*>(bias_s + col_a);
                    const float4* bb = reinterpret_cast<const float4*>(bias_s + col_b);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float4 a0 = ba[i], a1 = ba[4 + i], b0 = bb[i], b1 = bb[4 + i];
                        acc[2 * i] = make_float2(__uint_as_float(r0[4 * i]) + a0.x, __uint_as_float(r0[4 * i + 1]) + a0.y);
                        acc[2 * i + 1] = make_float2(__uint_as_float(r0[4 * i + 2]) + a0.z, __uint_as_float(r0[4 * i + 3]) + a0.w);
                        acc[8 + 2 * i] = make_float2(__uint_as_float(r1[4 * i]) + a1.x, __uint_as_float(r1[4 * i + 1]) + a1.y);
                        acc[8 + 2 * i + 1] = make_float2(__uint_as_float(r1[4 * i + 2]) + a1.z, __uint_as_float(r1[4 * i + 3]) + a1.w);
                        acc[16 + 2 * i] = make_float2(__uint_as_float(r2[4 * i]) + b0.x, __uint_as_float(r2[4 * i + 1]) + b0.y);
                        acc[16 + 2 * i + 1] = make_float2(__uint_as_float(r2[4 * i + 2]) + b0.z, __uint_as_float(r2[4 * i + 3]) + b0.w);
                        acc[24 + 2 * i] = make_float2(__uint_as_float(r3[4 * i]) + b1.x, __uint_as_float(r3[4 * i + 1]) + b1.y);
                        acc[24 + 2 * i + 1] = make_float2(__uint_as_float(r3[4 * i + 2]) + b1.z, __uint_as_float(r3[4 * i + 3]) + b1.w);
                    }
                }
                tc_fence_before_sync();
                mbar_arrive(&tmem_empty);
                // -------------------------------------------------------- tile epilogue (from registers)
                const int swz = row_in_tile & 7;
                if (MODE == kSwiGLU || MODE == kSiLU) {
                    constexpr int NV = MODE == kSwiGLU ? 16 : 32;  // float2 values this thread produces
                    float amax = 0.f;
#pragma unroll
                    for (int i = 0; i < NV; ++i) {
                        float2 h = make_float2(silu(acc[i].x), silu(acc[i].y));
                        if (MODE == kSwiGLU) h = __fmul2_rn(h, acc[16 + i]);
                        acc[i] = h;
                        amax = fmaxf(amax, fmaxf(fabsf(h.x), fabsf(h.y)));
                    }
                    float (*xchg)[kBM] = amax_xchg[tile_count & 1];
                    xchg[cq][row_in_tile] = amax;
                    if (leader) bulk_wait_read<0>();        // the group's previous store has read its staging rows
                    asm volatile("bar.sync %0, 128;" ::"r"(group_bar) : "memory");
                    if (MODE == kSwiGLU) {
                        amax = fmaxf(fmaxf(xchg[0][row_in_tile], xchg[1][row_in_tile]),
                                     fmaxf(xchg[2][row_in_tile], xchg[3][row_in_tile]));
                    } else {
                        amax = fmaxf(amax, xchg[cq ^ 1][row_in_tile]);
                    }
                    float inv1;
                    const uint32_t sf_byte = pow2_scale(amax, &inv1);
                    const float2 inv = make_float2(inv1, inv1);
                    uint8_t* box_row = out_q + (MODE == kSiLU ? (cq >> 1) * kOutBoxBytes : 0) + lane * 128;
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
                    // the hidden block's scale, repeated for its four slices, in the atom layout the next GEMM loads
                    const bool writer = MODE == kSwiGLU ? cq == 0 : (cq & 1) == 0;
                    if (row_ok && writer) {
                        const int hidden_blocks = MODE == kSwiGLU ? g.N / 256 : g.N / 128;
                        const int hb = MODE == kSwiGLU ? n0 / kBN : (n0 + cq * 64) / 128;
                        uint8_t* atom = g.out_sf + (m * hidden_blocks + hb) * kSfAtom;
                        *reinterpret_cast<uint32_t*>(atom + sf_row_offset(row_in_tile)) = sf_byte * 0x01010101u;
                    }
                } else {
                    uint8_t* box_row = out_q + cq * kOutBoxBytes + lane * 128;
                    const bool has_res = g.residual != nullptr;
                    if (!has_res) {
                        if (leader) bulk_wait_read<0>();
                        asm volatile("bar.sync %0, 128;" ::"r"(group_bar) : "memory");
                    } else if (ok && !mbar_wait_sleep(&res_full[quarter], tile_count & 1)) {
                        ok = false;
                    }
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
                // the group's rows are staged -> its leader hands them to TMA (rows past M are clipped by the tensor map)
                fence_proxy_async_smem();
                asm volatile("bar.sync %0, 128;" ::"r"(group_bar) : "memory");
                if (leader) {
                    const int x0 = MODE == kSwiGLU ? (n0 / kBN) * 128 : (MODE == kSiLU ? n0 : 2 * n0);
#pragma unroll
                    for (int b = 0; b < P::kOutBoxes; ++b)
                        tma_store_2d(&tmap_o, out_q + b * kOutBoxBytes, x0 + b * 128, m0 + quarter * 32);
                    bulk_commit();
                }
            }
        }
        if (leader) bulk_wait<0>();
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
// CTA-pair variant (cluster of two CTAs, tcgen05 cta_group::2).  A pair owns a 256 x 256 output tile: each CTA loads
// its own 128 rows of A with their scale atoms, one half (128 rows) of the weight tile and the scale atoms of the
// WHOLE weight tile (every CTA's tensor core scales all 256 output columns of its rows); the leader (even rank) issues
// 256 x 256 x 32 block-scaled MMAs that read A from each CTA's own shared memory and the weight halves from both,
// and the scale-factor copies into tensor memory in their two-CTA form (each CTA copies from its own shared memory
// into its own tensor memory).  A stage is 33.5 KB per CTA for 512 cycles of tensor-core time instead of 49.5 KB, and
// with a resident weight half of 64 KB the activation ring has seven stages.  Barriers as in the bf16 pair kernel: "full" lives in the leader and counts the bytes
// of both CTAs' loads; "empty" and "accumulator full" are signalled in both CTAs by multicast commits;
// "accumulator empty" collects one arrival per epilogue warp of both CTAs in the leader.
// ------------------------------------------------------------------------------------------------
constexpr uint32_t kBHalfBytes = kBBytes / 2;                 // 16 KB: this CTA's half of the weight tile
constexpr uint32_t kPeerMask = 0xFEFFFFFFu;                   // shared::cluster address of the pair's even CTA
constexpr int kEpiWarps = kEpiThreads / 32;

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* m, int32_t c0, int32_t c1, uint64_t* leader_bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(smem_dst)),
        "l"(m), "r"(smem_u32(leader_bar) & kPeerMask), "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void mma_mxf8_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate,
                                                 uint32_t sfa_tmem, uint32_t sfb_tmem) {
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::mxf8f6f4.block_scale [%0], %1, %2, %3, [%5], [%6], p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(sfa_tmem), "r"(sfb_tmem)
        : "memory");
}
// each CTA of the pair copies the atom at this offset of ITS shared memory into ITS tensor memory
__device__ __forceinline__ void tc_cp_32x128b_warpx4_pair(uint32_t taddr, uint64_t smem_desc) {
    asm volatile("tcgen05.cp.cta_group::2.32x128b.warpx4 [%0], %1;" ::"r"(taddr), "l"(smem_desc) : "memory");
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

template <int MODE, bool B_RES>
struct PairPlan {
    static constexpr int kOutBoxes = MODE == kSwiGLU ? 1 : (MODE == kSiLU ? 2 : 4);
    static constexpr uint32_t kOutBytes = kOutBoxes * kOutBoxBytes;
    static constexpr int kStagesN = B_RES ? (MODE == kSiLU ? 6 : 7) : 4;
    // A tile (+ weight half) + scale atoms of A (+ of the whole weight tile), padded to a multiple of 1 KB
    static constexpr uint32_t kStageBytesN = B_RES ? kABytes + 1024 : kABytes + kBHalfBytes + 2048;
    static constexpr uint32_t kStageTx = B_RES ? kABytes + kSfaBytes : kABytes + kBHalfBytes + kSfaBytes + kSfbBytes;
    static constexpr size_t tiles_bytes(int k_blocks) {
        return (B_RES ? static_cast<size_t>(k_blocks) * (kBHalfBytes + kSfbBytes) : 0) + static_cast<size_t>(kStagesN) * kStageBytesN +
               kOutBytes;
    }
};

template <int MODE, bool B_RES>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
mx_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                    const __grid_constant__ CUtensorMap tmap_o, const __grid_constant__ CUtensorMap tmap_r, const GemmArgs g) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[kMaxStages + 1];   // used in the leader only
    __shared__ uint64_t empty_bar[kMaxStages + 1];
    __shared__ uint64_t b_full;                     // used in the leader only
    __shared__ uint64_t res_full[4];
    __shared__ uint64_t tmem_full;
    __shared__ uint64_t tmem_empty;                 // used in the leader only
    __shared__ uint32_t tmem_base_slot;
    __shared__ __align__(16) float bias_s[kBN];
    __shared__ float amax_xchg[2][4][kBM];
    __shared__ int s_abort;

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();           // 0 = leader
    const int pair = blockIdx.x >> 1;
    const int n_pairs = gridDim.x >> 1;

    const int64_t m_tiles = (g.M + 2 * kBM - 1) / (2 * kBM);     // row tiles of 256 rows, 128 per CTA
    const int n_tiles = g.N / kBN;
    const int k_blocks = g.K / kBK;
    using P = PairPlan<MODE, B_RES>;
    constexpr int STAGES = P::kStagesN;
    constexpr uint32_t STAGE_BYTES = P::kStageBytesN;
    uint8_t* b_res = smem;                                                       // [k_blocks][16 KB]: this CTA's weight rows
    uint8_t* sfb_res = smem + static_cast<size_t>(k_blocks) * kBHalfBytes;       // [k_blocks][1 KB]: scale atoms of all 256 rows
    uint8_t* ring = B_RES ? smem + static_cast<size_t>(k_blocks) * (kBHalfBytes + kSfbBytes) : smem;
    uint8_t* out_s = ring + static_cast<size_t>(STAGES) * STAGE_BYTES;
    constexpr uint32_t kSfaInStage = B_RES ? kABytes : kABytes + kBHalfBytes;
    constexpr uint32_t kSfbInStage = kSfaInStage + kSfaBytes;

    // a pair keeps one column tile for its whole life where there are enough pairs, and walks down the row tiles
    int n_first, n_step, row_first, row_step;
    bool active = true;
    if (n_tiles <= n_pairs) {
        row_step = n_pairs / n_tiles;
        n_first = pair % n_tiles;
        row_first = pair / n_tiles;
        n_step = 0x40000000;
        active = row_first < row_step;
    } else {
        row_step = 1;
        row_first = 0;
        n_first = pair;
        n_step = n_pairs;
    }

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        mbar_init(&b_full, 1);
        for (int q = 0; q < 4; ++q) mbar_init(&res_full[q], 1);
        mbar_init(&tmem_full, 1);
        mbar_init(&tmem_empty, 2 * kEpiWarps);
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

    if (warp == 0) {
        // ---------------------------------------------------------------- producer (both CTAs)
        if (lane == 0 && active) {
            tma_prefetch_desc(&tmap_a);
            tma_prefetch_desc(&tmap_b);
            tma_prefetch_desc(&tmap_sfa);
            tma_prefetch_desc(&tmap_sfb);
            uint32_t it = 0;
            bool ok = true;
            for (int n = n_first; n < n_tiles && ok; n += n_step) {
                const int n0 = n * kBN;
                const int sfb_atom0 = (n0 / 128) * k_blocks;          // atoms of weight block n0 / 128; the next block follows k_blocks later
                if (B_RES) {
                    if (it > 0) {  // the previous column tile's MMAs must have finished reading the resident tiles
                        const uint32_t last = it - 1;
                        if (!mbar_wait_sleep(&empty_bar[last % STAGES], (last / STAGES) & 1)) { ok = false; break; }
                    }
                    if (rank == 0) mbar_expect_tx(&b_full, 2u * static_cast<uint32_t>(k_blocks) * (kBHalfBytes + kSfbBytes));
                    for (int kb = 0; kb < k_blocks; ++kb) {
                        tma_load_2d_pair(b_res + static_cast<size_t>(kb) * kBHalfBytes, &tmap_b, kb * kBK, n0 + static_cast<int>(rank) * 128, &b_full);
                        tma_load_2d_pair(sfb_res + kb * kSfbBytes, &tmap_sfb, 0, 2 * (sfb_atom0 + kb), &b_full);
                        tma_load_2d_pair(sfb_res + kb * kSfbBytes + kSfAtom, &tmap_sfb, 0, 2 * (sfb_atom0 + k_blocks + kb), &b_full);
                    }
                }
                for (int64_t m = row_first; m < m_tiles && ok; m += row_step) {
                    const int64_t tile128 = 2 * m + rank;                 // this CTA's 128-row tile
                    const int m0 = static_cast<int>(tile128) * kBM;
                    for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                        const uint32_t s = it % STAGES;
                        const uint32_t ph = (it / STAGES) & 1;
                        if (!mbar_wait_sleep(&empty_bar[s], ph ^ 1) || *reinterpret_cast<volatile int*>(&s_abort)) {
                            ok = false;
                            break;
                        }
                        uint8_t* stage = ring + static_cast<size_t>(s) * STAGE_BYTES;
                        if (rank == 0) mbar_expect_tx(&full_bar[s], 2u * P::kStageTx);   // the bytes of both CTAs
                        tma_load_2d_pair(stage, &tmap_a, kb * kBK, m0, &full_bar[s]);
                        tma_load_2d_pair(stage + kSfaInStage, &tmap_sfa, 0, static_cast<int32_t>(2 * (tile128 * k_blocks + kb)), &full_bar[s]);
                        if (!B_RES) {
                            tma_load_2d_pair(stage + kABytes, &tmap_b, kb * kBK, n0 + static_cast<int>(rank) * 128, &full_bar[s]);
                            tma_load_2d_pair(stage + kSfbInStage, &tmap_sfb, 0, 2 * (sfb_atom0 + kb), &full_bar[s]);
                            tma_load_2d_pair(stage + kSfbInStage + kSfAtom, &tmap_sfb, 0, 2 * (sfb_atom0 + k_blocks + kb), &full_bar[s]);
                        }
                    }
                }
            }
            if (!ok) {
                s_abort = 1;
                if (g.status != nullptr) atomicExch(g.status, 1);
            }
        }
    } else if (warp == 1) {
        // ---------------------------------------------------------------- MMA issuer (leader only)
        if (lane == 0 && rank == 0 && active) {
            const uint64_t desc0 = umma_desc_sw128(0, 1024, 16);
            const uint64_t sf_desc0 = umma_desc_noswizzle(0, 128, 0);
            const uint32_t ring_lo = (smem_u32(ring) & 0x3FFFFu) >> 4;
            const uint32_t bres_lo = B_RES ? (smem_u32(b_res) & 0x3FFFFu) >> 4 : 0u;
            const uint32_t sfbres_lo = B_RES ? (smem_u32(sfb_res) & 0x3FFFFu) >> 4 : 0u;
            uint32_t s = 0, ph = 0, b_phase = 0, tile = 0, it = 0;
            bool ok = true;
            for (int n = n_first; n < n_tiles && ok; n += n_step) {
                if (B_RES) {
                    if (!mbar_wait_sleep(&b_full, b_phase)) { ok = false; break; }
                    b_phase ^= 1;
                    tc_fence_after_sync();
                    for (int kb = 0; kb < k_blocks; ++kb) {
                        const uint32_t src = sfbres_lo + static_cast<uint32_t>(kb) * (kSfbBytes >> 4);
                        tc_cp_32x128b_warpx4_pair(tmem_base + kTmemSfbRes + kb * 8, sf_desc0 + src);
                        tc_cp_32x128b_warpx4_pair(tmem_base + kTmemSfbRes + kb * 8 + 4, sf_desc0 + src + (kSfAtom >> 4));
                    }
                }
                for (int64_t m = row_first; m < m_tiles && ok; m += row_step, ++tile) {
                    if (!mbar_wait_sleep(&tmem_empty, (tile & 1) ^ 1)) { ok = false; break; }
                    tc_fence_after_sync();
                    for (int kb = 0; kb < k_blocks; ++kb, ++it) {
                        if (!mbar_wait_sleep(&full_bar[s], ph)) { ok = false; break; }
                        tc_fence_after_sync();
                        const uint32_t a_lo = ring_lo + s * (STAGE_BYTES >> 4);
                        const uint32_t b_lo = B_RES ? bres_lo + static_cast<uint32_t>(kb) * (kBHalfBytes >> 4) : a_lo + (kABytes >> 4);
                        const uint32_t sfa_lo = a_lo + (kSfaInStage >> 4);
                        const uint32_t sfb_lo = a_lo + (kSfbInStage >> 4);
                        const uint32_t t_sfa = tmem_base + kTmemSf + (it & 1) * kSfSlotCols;
                        const uint32_t t_sfb = B_RES ? tmem_base + kTmemSfbRes + kb * 8 : t_sfa + 4;
                        tc_cp_32x128b_warpx4_pair(t_sfa, sf_desc0 + sfa_lo);
                        if (!B_RES) {
                            tc_cp_32x128b_warpx4_pair(t_sfb, sf_desc0 + sfb_lo);
                            tc_cp_32x128b_warpx4_pair(t_sfb + 4, sf_desc0 + sfb_lo + (kSfAtom >> 4));
                        }
                        const uint64_t da = desc0 + a_lo;
                        const uint64_t db = desc0 + b_lo;
#pragma unroll
                        for (int k = 0; k < kBK / 32; ++k)
                            mma_mxf8_ss_pair(tmem_base, da + 2 * k, db + 2 * k, umma_idesc_mx(2 * kBM, kBN, k, k), (kb > 0 || k > 0) ? 1u : 0u,
                                             t_sfa, t_sfb);
                        tc_commit_pair(&empty_bar[s]);
                        if (++s == STAGES) {
                            s = 0;
                            ph ^= 1;
                        }
                    }
                    if (ok) tc_commit_pair(&tmem_full);
                }
            }
            if (!ok) {
                s_abort = 1;
                if (g.status != nullptr) atomicExch(g.status, 1);
            }
        }
    } else {
        // ---------------------------------------------------------------- epilogue (both CTAs, own 128 rows)
        const int et = threadIdx.x - 64;
        const int cq = et >> 7;
        const int quarter = warp & 3;
        const int row_in_tile = quarter * 32 + lane;
        const uint32_t lane_addr = static_cast<uint32_t>(quarter * 32) << 16;
        const int col_a = MODE == kSwiGLU ? cq * 32 : cq * 64;
        const int col_b = MODE == kSwiGLU ? 128 + cq * 32 : cq * 64 + 32;
        const bool leader = cq == 0 && lane == 0;
        const uint32_t group_bar = 2 + quarter;
        uint8_t* out_q = out_s + quarter * 4096;
        uint32_t tile_count = 0;
        bool ok = true;

        for (int n = n_first; n < n_tiles && active; n += n_step) {
            const int n0 = n * kBN;
            asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
            if (et < kBN) bias_s[et] = g.bias != nullptr ? g.bias[n0 + et] : 0.f;
            asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");

            for (int64_t m = row_first; m < m_tiles; m += row_step, ++tile_count) {
                const int64_t tile128 = 2 * m + rank;
                const int64_t row = tile128 * kBM + row_in_tile;
                const bool row_ok = row < g.M;
                const int m0 = static_cast<int>(tile128) * kBM;
                const bool rows_here = static_cast<int64_t>(m0) + quarter * 32 < g.M;      // any row of this group inside the matrix
                if (MODE == kLinear && g.residual != nullptr && leader) {
                    bulk_wait_read<0>();
                    if (rows_here) {
                        mbar_expect_tx(&res_full[quarter], P::kOutBoxes * 4096u);
#pragma unroll
                        for (int b = 0; b < P::kOutBoxes; ++b)
                            tma_load_2d(out_q + b * kOutBoxBytes, &tmap_r, 2 * n0 + b * 128, m0 + quarter * 32, &res_full[quarter]);
                    } else {
                        mbar_arrive(&res_full[quarter]);       // nothing to fetch: complete the phase by hand
                    }
                }
                if (ok) {   // one lane polls, the warp follows
                    int passed = 1;
                    if (lane == 0) passed = mbar_wait_sleep(&tmem_full, tile_count & 1) ? 1 : 0;
                    if (__shfl_sync(0xffffffffu, passed, 0) == 0) ok = false;
                }
                tc_fence_after_sync();
                float2 acc[32];
                const uint32_t t0 = tmem_base + lane_addr;
                {
                    uint32_t r0[16], r1[16], r2[16], r3[16];
                    tmem_ld_x16(t0 + col_a, r0);
                    tmem_ld_x16(t0 + col_a + 16, r1);
                    tmem_ld_x16(t0 + col_b, r2);
                    tmem_ld_x16(t0 + col_b + 16, r3);
                    tc_wait_ld(r0);
                    tc_wait_ld(r1);
                    tc_wait_ld(r2);
                    tc_wait_ld(r3);
                    // the warp holds its share of the accumulator in registers: hand it back to the leader
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) mbar_arrive_leader(&tmem_empty);
                    const float4* ba = reinterpret_cast<const float4*>(bias_s + col_a);
                    const float4* bb = reinterpret_cast<const float4*>(bias_s + col_b);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float4 a0 = ba[i], a1 = ba[4 + i], b0 = bb[i], b1 = bb[4 + i];
                        acc[2 * i] = make_float2(__uint_as_float(r0[4 * i]) + a0.x, __uint_as_float(r0[4 * i + 1]) + a0.y);
                        acc[2 * i + 1] = make_float2(__uint_as_float(r0[4 * i + 2]) + a0.z, __uint_as_float(r0[4 * i + 3]) + a0.w);
                        acc[8 + 2 * i] = make_float2(__uint_as_float(r1[4 * i]) + a1.x, __uint_as_float(r1[4 * i + 1]) + a1.y);
                        acc[8 + 2 * i + 1] = make_float2(__uint_as_float(r1[4 * i + 2]) + a1.z, __uint_as_float(r1[4 * i + 3]) + a1.w);
                        acc[16 + 2 * i] = make_float2(__uint_as_float(r2[4 * i]) + b0.x, __uint_as_float(r2[4 * i + 1]) + b0.y);
                        acc[16 + 2 * i + 1] = make_float2(__uint_as_float(r2[4 * i + 2]) + b0.z, __uint_as_float(r2[4 * i + 3]) + b0.w);
                        acc[24 + 2 * i] = make_float2(__uint_as_float(r3[4 * i]) + b1.x, __uint_as_float(r3[4 * i + 1]) + b1.y);
                        acc[24 + 2 * i + 1] = make_float2(__uint_as_float(r3[4 * i + 2]) + b1.z, __uint_as_float(r3[4 * i + 3]) + b1.w);
                    }
                }
                const int swz = row_in_tile & 7;
                if (MODE == kSwiGLU || MODE == kSiLU) {
                    constexpr int NV = MODE == kSwiGLU ? 16 : 32;
                    float amax = 0.f;
#pragma unroll
                    for (int i = 0; i < NV; ++i) {
                        float2 h = make_float2(silu(acc[i].x), silu(acc[i].y));
                        if (MODE == kSwiGLU) h = __fmul2_rn(h, acc[16 + i]);
                        acc[i] = h;
                        amax = fmaxf(amax, fmaxf(fabsf(h.x), fabsf(h.y)));
                    }
                    float (*xchg)[kBM] = amax_xchg[tile_count & 1];
                    xchg[cq][row_in_tile] = amax;
                    if (leader) bulk_wait_read<0>();
                    asm volatile("bar.sync %0, 128;" ::"r"(group_bar) : "memory");
                    if (MODE == kSwiGLU) {
                        amax = fmaxf(fmaxf(xchg[0][row_in_tile], xchg[1][row_in_tile]),
                                     fmaxf(xchg[2][row_in_tile], xchg[3][row_in_tile]));
                    } else {
                        amax = fmaxf(amax, xchg[cq ^ 1][row_in_tile]);
                    }
                    float inv1;
                    const uint32_t sf_byte = pow2_scale(amax, &inv1);
                    const float2 inv = make_float2(inv1, inv1);
                    uint8_t* box_row = out_q + (MODE == kSiLU ? (cq >> 1) * kOutBoxBytes : 0) + lane * 128;
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
                    const bool writer = MODE == kSwiGLU ? cq == 0 : (cq & 1) == 0;
                    if (row_ok && writer) {
                        const int hidden_blocks = MODE == kSwiGLU ? g.N / 256 : g.N / 128;
                        const int hb = MODE == kSwiGLU ? n0 / kBN : (n0 + cq * 64) / 128;
                        uint8_t* atom = g.out_sf + (tile128 * hidden_blocks + hb) * kSfAtom;
                        *reinterpret_cast<uint32_t*>(atom + sf_row_offset(row_in_tile)) = sf_byte * 0x01010101u;
                    }
                } else {
                    uint8_t* box_row = out_q + cq * kOutBoxBytes + lane * 128;
                    const bool has_res = g.residual != nullptr;
                    if (!has_res) {
                        if (leader) bulk_wait_read<0>();
                        asm volatile("bar.sync %0, 128;" ::"r"(group_bar) : "memory");
                    } else if (ok && !mbar_wait_sleep(&res_full[quarter], tile_count & 1)) {
                        ok = false;
                    }
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        uint4* slot = reinterpret_cast<uint4*>(box_row + ((c ^ swz) << 4));
                        float2 v[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) v[e] = acc[4 * c + e];
                        if (has_res && rows_here) {
                            float2 rr[4];
                            Vec16<__nv_bfloat16>::unpack2(*slot, rr);
#pragma unroll
                            for (int e = 0; e < 4; ++e) v[e] = __fadd2_rn(v[e], rr[e]);
                        }
                        *slot = Vec16<__nv_bfloat16>::pack2(v);
                    }
                }
                fence_proxy_async_smem();
                asm volatile("bar.sync %0, 128;" ::"r"(group_bar) : "memory");
                if (leader) {
                    const int x0 = MODE == kSwiGLU ? (n0 / kBN) * 128 : (MODE == kSiLU ? n0 : 2 * n0);
                    if (rows_here) {
#pragma unroll
                        for (int b = 0; b < P::kOutBoxes; ++b)
                            tma_store_2d(&tmap_o, out_q + b * kOutBoxBytes, x0 + b * 128, m0 + quarter * 32);
                    }
                    bulk_commit();
                }
            }
        }
        if (leader) bulk_wait<0>();
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

// ------------------------------------------------------------------------------------------------
// activation quantisation: bf16 [M, K] -> e4m3 [M, K] + scale atoms [ceil(M / 128), K / 128, 512]
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
quant_act_mx_kernel(const uint4* __restrict__ x, uint2* __restrict__ q, uint8_t* __restrict__ sf, int64_t n_blocks, int k_blocks) {
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
    float inv;
    const uint32_t byte = pow2_scale(amax, &inv);
    if (ok) {
        uint2 w;
        w.x = pack_e4m3x4(f[0] * inv, f[1] * inv, f[2] * inv, f[3] * inv);
        w.y = pack_e4m3x4(f[4] * inv, f[5] * inv, f[6] * inv, f[7] * inv);
        q[block * 16 + sub] = w;
        if (sub == 0) {
            const int64_t row = block / k_blocks;
            const int kb = static_cast<int>(block - row * k_blocks);
            uint8_t* atom = sf + ((row >> 7) * k_blocks + kb) * kSfAtom;
            *reinterpret_cast<uint32_t*>(atom + sf_row_offset(static_cast<int>(row & 127))) = byte * 0x01010101u;
        }
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
bool make_tmap_bytes(CUtensorMap* map, const void* base, uint64_t k_bytes, uint64_t rows, uint64_t pitch_bytes, uint32_t box_rows) {
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
int launch_gemm_impl(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, const CUtensorMap& tr, const GemmArgs& g,
                     cudaStream_t stream) {
    using P = Plan<MODE, B_RES>;
    const DeviceInfo& dev = device_info();
    const size_t smem = P::tiles_bytes(g.K / kBK) + 1024;
    static bool attr_set[64] = {};
    if (!attr_set[dev.index]) {
        cudaFuncSetAttribute(mx_gemm_kernel<MODE, B_RES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(P::tiles_bytes(4) + 1024));
        attr_set[dev.index] = true;
    }
    const int64_t m_tiles = (g.M + kBM - 1) / kBM;
    const int n_tiles = g.N / kBN;
    int64_t grid = dev.sm_count;
    if (n_tiles <= grid) {
        int64_t walkers = grid / n_tiles;
        if (walkers > m_tiles) walkers = m_tiles;
        grid = walkers * n_tiles;
    }
    mx_gemm_kernel<MODE, B_RES><<<static_cast<unsigned>(grid), kThreads, smem, stream>>>(ta, tb, to, tr, g);
    count_launch();
    return launch_status();
}

template <int MODE>
int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& to, const CUtensorMap& tr, const GemmArgs& g,
                cudaStream_t stream) {
    if (MODE != kLinear && g.K <= 4 * kBK) return launch_gemm_impl<MODE, true>(ta, tb, to, tr, g, stream);
    return launch_gemm_impl<MODE, false>(ta, tb, to, tr, g, stream);
}

// scale atoms as a 2-D byte tensor [2 * atoms, 256]: one atom = a box of 2 rows, no swizzle
bool make_tmap_atoms(CUtensorMap* map, const void* base, uint64_t atoms) {
    PFN_cuTensorMapEncodeTiled_v12000 fn = encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[2] = {256, 2 * atoms};
    const cuuint64_t strides[1] = {256};
    const cuuint32_t box[2] = {256, 2};
    const cuuint32_t elem[2] = {1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int MODE, bool B_RES>
int launch_pair_impl(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa, const CUtensorMap& tsb, const CUtensorMap& to,
                     const CUtensorMap& tr, const GemmArgs& g, cudaStream_t stream) {
    using P = PairPlan<MODE, B_RES>;
    const DeviceInfo& dev = device_info();
    const size_t smem = P::tiles_bytes(g.K / kBK) + 1024;
    static bool attr_set[64] = {};
    if (!attr_set[dev.index]) {
        cudaFuncSetAttribute(mx_gemm_pair_kernel<MODE, B_RES>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             static_cast<int>(P::tiles_bytes(4) + 1024));
        attr_set[dev.index] = true;
    }
    const int64_t m_tiles = (g.M + 2 * kBM - 1) / (2 * kBM);
    const int n_tiles = g.N / kBN;
    int64_t pairs = dev.sm_count / 2;
    if (n_tiles <= pairs) {
        int64_t walkers = pairs / n_tiles;
        if (walkers > m_tiles) walkers = m_tiles;
        pairs = walkers * n_tiles;
    }
    mx_gemm_pair_kernel<MODE, B_RES><<<static_cast<unsigned>(2 * pairs), kThreads, smem, stream>>>(ta, tb, tsa, tsb, to, tr, g);
    count_launch();
    return launch_status();
}

template <int MODE>
int launch_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa, const CUtensorMap& tsb, const CUtensorMap& to,
                const CUtensorMap& tr, const GemmArgs& g, cudaStream_t stream) {
    if (MODE != kLinear && g.K <= 4 * kBK) return launch_pair_impl<MODE, true>(ta, tb, tsa, tsb, to, tr, g, stream);
    return launch_pair_impl<MODE, false>(ta, tb, tsa, tsb, to, tr, g, stream);
}

// CTA pairs serve the streamed-weight case (K > 512, e.g. the down projection), where halving the weight bytes per CTA
// relieves the L2 feed: measured 0.279 against 0.289 ms at 262 144 x 2048 -> 512.  With a resident weight tile
// (K <= 512) the single-CTA kernel is the faster one (0.614 against 0.684 ms at 262 144 x 512 -> 4096): both are bound
// by the hand-off of the single accumulator between the K loop and the epilogue, not by the ring, and pairs leave 20 of
// the 148 SMs idle at 16 column tiles.  TB200_MX_PAIR=0 / =2 in the environment force the single-CTA / the pair kernel.
bool use_pairs(int64_t M, int32_t K, int mode) {
    static const int choice = [] {
        const char* e = std::getenv("TB200_MX_PAIR");
        return e == nullptr ? 1 : (e[0] == '0' ? 0 : (e[0] == '2' ? 2 : 1));
    }();
    if (choice == 0 || M <= kBM) return false;
    if (choice == 2) return true;
    return mode == kLinear || K > 4 * kBK;
}

}  // namespace
}  // namespace tb200

extern "C" int64_t tb200_mx_scale_bytes(int64_t rows, int32_t K) {
    if (rows < 0 || K < 128 || K % 128 != 0) return 0;
    return ((rows + 127) / 128) * (K / 128) * static_cast<int64_t>(tb200::kSfAtom);
}

extern "C" int tb200_quant_act_mx(const void* x_bf16, void* x_fp8, uint8_t* scale_atoms, int64_t M, int32_t K, void* stream) {
    using namespace tb200;
    if (M < 0 || K < 128 || K % 128 != 0) return TB200_ERR_SHAPE;
    if (M == 0) return TB200_OK;
    if (x_bf16 == nullptr || x_fp8 == nullptr || scale_atoms == nullptr) return TB200_ERR_NULL;
    if (!aligned16(x_bf16) || !aligned16(x_fp8) || !aligned16(scale_atoms)) return TB200_ERR_ALIGN;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    const int64_t n_blocks = M * (K / 128);
    const int64_t grid = (n_blocks * 16 + 255) / 256;
    if (grid > 0x7FFFFFFFll) return TB200_ERR_SHAPE;
    quant_act_mx_kernel<<<static_cast<unsigned>(grid), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const uint4*>(x_bf16), static_cast<uint2*>(x_fp8), scale_atoms, n_blocks, K / 128);
    count_launch();
    return launch_status();
}

extern "C" int tb200_mx_gemm(const void* a_fp8, const uint8_t* a_scale_atoms, const void* b_fp8, const uint8_t* b_scale_atoms,
                             const float* bias, const void* residual, void* out, uint8_t* out_scale_atoms, int64_t M, int32_t N,
                             int32_t K, int32_t mode, int32_t* status_word, void* stream) {
    using namespace tb200;
    if (M < 0 || N < 256 || N % 256 != 0 || K < 128 || K % 128 != 0 || K > 8192) return TB200_ERR_SHAPE;
    if (mode < 0 || mode > 2) return TB200_ERR_UNSUPPORTED;
    if (M == 0) return TB200_OK;
    if (a_fp8 == nullptr || a_scale_atoms == nullptr || b_fp8 == nullptr || b_scale_atoms == nullptr || out == nullptr)
        return TB200_ERR_NULL;
    if (mode != kLinear && out_scale_atoms == nullptr) return TB200_ERR_NULL;
    if (mode != kLinear && residual != nullptr) return TB200_ERR_UNSUPPORTED;
    if (!aligned16(a_fp8) || !aligned16(b_fp8) || !aligned16(out) || !aligned16(a_scale_atoms) || !aligned16(b_scale_atoms) ||
        (residual != nullptr && !aligned16(residual)) || (out_scale_atoms != nullptr && !aligned16(out_scale_atoms)))
        return TB200_ERR_ALIGN;
    if (M > 0x7FFFFF00ll) return TB200_ERR_SHAPE;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    CUtensorMap ta, tb;
    if (!make_tmap_bytes(&ta, a_fp8, static_cast<uint64_t>(K), static_cast<uint64_t>(M), static_cast<uint64_t>(K), kBM) ||
        !make_tmap_bytes(&tb, b_fp8, static_cast<uint64_t>(K), static_cast<uint64_t>(N), static_cast<uint64_t>(K), kBN))
        return TB200_ERR_DRIVER;
    const uint64_t out_row_bytes = mode == kSwiGLU ? static_cast<uint64_t>(N) / 2 : (mode == kSiLU ? static_cast<uint64_t>(N) : 2ull * N);
    CUtensorMap to, tr;
    // output and residual move in boxes of 32 rows x 128 bytes: one per epilogue group (a TMEM lane quarter)
    if (!make_tmap_bytes(&to, out, out_row_bytes, static_cast<uint64_t>(M), out_row_bytes, 32)) return TB200_ERR_DRIVER;
    if (!make_tmap_bytes(&tr, residual != nullptr ? residual : out, out_row_bytes, static_cast<uint64_t>(M), out_row_bytes, 32))
        return TB200_ERR_DRIVER;
    GemmArgs g{};
    g.sfa = a_scale_atoms;
    g.sfb = b_scale_atoms;
    g.bias = bias;
    g.residual = static_cast<const __nv_bfloat16*>(residual);
    g.out = out;
    g.out_sf = out_scale_atoms;
    g.status = status_word;
    g.M = M;
    g.N = N;
    g.K = K;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (use_pairs(M, K, mode)) {
        CUtensorMap tbh, tsa, tsb;
        const uint64_t k_blocks = static_cast<uint64_t>(K / kBK);
        if (!make_tmap_bytes(&tbh, b_fp8, static_cast<uint64_t>(K), static_cast<uint64_t>(N), static_cast<uint64_t>(K), 128) ||
            !make_tmap_atoms(&tsa, a_scale_atoms, static_cast<uint64_t>((M + 127) / 128) * k_blocks) ||
            !make_tmap_atoms(&tsb, b_scale_atoms, static_cast<uint64_t>(N / 128) * k_blocks))
            return TB200_ERR_DRIVER;
        if (mode == kSwiGLU) return launch_pair<kSwiGLU>(ta, tbh, tsa, tsb, to, tr, g, s);
        if (mode == kSiLU) return launch_pair<kSiLU>(ta, tbh, tsa, tsb, to, tr, g, s);
        return launch_pair<kLinear>(ta, tbh, tsa, tsb, to, tr, g, s);
    }
    if (mode == kSwiGLU) return launch_gemm<kSwiGLU>(ta, tb, to, tr, g, s);
    if (mode == kSiLU) return launch_gemm<kSiLU>(ta, tb, to, tr, g, s);
    return launch_gemm<kLinear>(ta, tb, to, tr, g, s);
}
