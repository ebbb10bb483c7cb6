// Sequence tokenizer in one kernel for sm_100a:
//     x[r, :]      = concat_f table_f[clamp(ids[f, r])]                       (row gather, K = n_feat * emb columns)
//     p[r, :]      = x[r, :] W^T + bias                                       (tcgen05 GEMM, fp32 accumulators in TMEM)
//     tokens[r, :] = LayerNorm(SiLU(p[r, :])) + table_a[ids_a[r]] (+ table_b[ids_b[r]])
//     normed[r, :] = RMSNorm(tokens[r, :])
// i.e. `nn.Embedding` lookups, `torch.cat`, `Linear -> SiLU -> LayerNorm`, the time-bucket and position rows
// (src/taac2026/infrastructure/modeling/tokenizers.py:156-190) and the `attn_norm` of the first OneTrans block
// (experiments/onetrans/model.py:106), without the [rows, K] and [rows, N] intermediates ever reaching HBM:
// table rows come in once, `normed` goes out once, and `tokens` only for the rows a caller keeps (row_dst).
//
// A cluster of two CTAs owns a tile of 128 rows and splits the model width N (256 or 512 columns): each CTA keeps its
// N / 2 rows of W resident in shared memory, gathers the tile's rows (the second CTA's reads of a table row are
// served by the L2), runs its own tcgen05 MMAs (128 x N/2 x 16 per instruction) into one of two accumulator buffers
// in TMEM, and finishes its half of every row; the two halves of a row's statistics meet through distributed
// shared memory.  A thread owns one row and N / 8 columns, so the part of a row it keeps across the statistics is
// 32 registers at N = 512.  Each CTA has sixteen warps that all do the same work; per tile, in every thread:
//   gather    16-byte cp.async copies of table rows for the tile two ahead into the free stage of a two-stage ring
//             of A tiles, in the 128-byte-swizzled K-major layout the tensor core reads (a group of lanes copies
//             one row, so every instruction moves whole rows); a tile later: wait for the own copies, proxy fence,
//             arrive on the stage's "full" barrier
//   MMA       one thread issues the MMAs of the NEXT tile into the other accumulator buffer at the top of the
//             iteration, so they run under the whole epilogue of this tile
//   pass 1    this tile's accumulator columns go from TMEM to registers as bf16 SiLU values
//   rest      LayerNorm statistics (exact centred variance: local mean and centred sum of squares per thread,
//             combined over the row's eight column groups, four of them written by the other CTA), normalise, add the
//             table rows with one rounding per sum like tensor additions, RMS statistics the same way, the kept
//             `tokens` rows straight to global memory, `normed` through the warp's own staging box and a TMA store.
// The two exchanges per tile are cluster barriers; every thread of both CTAs walks the same tile list, so they always
// meet.  Every mbarrier wait is bounded; a warp whose wait gives up raises the status word and keeps walking, so
// nothing is left waiting for it.  No TMA load carries multicast.
#include <cudaTypedefs.h>

#include "tb200_common.cuh"
#include "tb200_ptx.cuh"

namespace tb200 {
void count_launch();

namespace {

constexpr int kRows = 128;                       // rows per CTA and tile
constexpr int kWarps = 16;
constexpr int kThreads = kWarps * 32;            // 512: sixteen warps leave 128 registers per thread
constexpr int kMaxFeat = 8;
constexpr int kMaxKBlocks = 2;                   // K <= 128
constexpr int kAStages = 2;
constexpr uint32_t kKBlockBytes = kRows * 128;   // one 64-column K block of an A tile: 16 KB
constexpr uint32_t kAStageBytes = kMaxKBlocks * kKBlockBytes;
constexpr uint32_t kBoxBytes = 32 * 128;         // staging box of an epilogue warp: 32 rows x 64 bf16
constexpr uint32_t kWait = 1u << 20;

struct TPArgs {
    const __nv_bfloat16* table[kMaxFeat];   // nullptr: the feature has no table (zeros)
    int64_t table_rows[kMaxFeat];
    const int64_t* ids;                      // [n_feat, rows]
    const float* bias;                       // [N] or nullptr
    const __nv_bfloat16* ln_gamma;
    const __nv_bfloat16* ln_beta;
    const __nv_bfloat16* rms_gamma;
    const __nv_bfloat16* table_a;
    const __nv_bfloat16* table_b;            // or nullptr
    const int64_t* ids_a;
    const int64_t* ids_b;
    const int32_t* row_dst;                  // or nullptr: tokens row r = input row r
    __nv_bfloat16* tokens;
    int32_t* status;
    int64_t rows, rows_a, rows_b, rows_out;
    int32_t n_feat, emb, k_blocks;
    float ln_eps, rms_eps;
};

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// shared::cluster address of the same variable in the CTA of rank `peer`
__device__ __forceinline__ uint32_t map_to_peer(uint32_t local_addr, uint32_t peer) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local_addr), "r"(peer));
    return r;
}
__device__ __forceinline__ void st_cluster_f2(uint32_t addr, float a, float b) {
    asm volatile("st.shared::cluster.v2.f32 [%0], {%1, %2};" ::"r"(addr), "f"(a), "f"(b) : "memory");
}
__device__ __forceinline__ void st_cluster_f1(uint32_t addr, float a) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(a) : "memory");
}
// bounded wait that also acquires the other CTA's writes made before its arrival
__device__ __forceinline__ bool wait_cluster(uint64_t* bar, uint32_t parity, uint32_t limit) {
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.acquire.cluster.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(ok)
            : "r"(smem_u32(bar)), "r"(parity)
            : "memory");
        if (ok) return true;
    }
    return false;
}
__device__ __forceinline__ void cp_async16(uint32_t smem_dst, const void* gmem_src, uint32_t src_bytes) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(smem_dst), "l"(gmem_src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ float2 silu2(float2 x) {   // h * tanh(h) + h, h = x / 2
    const float2 h = __fmul2_rn(x, make_float2(0.5f, 0.5f));
    float2 t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t.x) : "f"(h.x));
    asm("tanh.approx.f32 %0, %1;" : "=f"(t.y) : "f"(h.y));
    return __ffma2_rn(h, t, h);
}
__device__ __forceinline__ uint32_t pack_bf16x2(float2 v) {
    const __nv_bfloat162 h = __float22bfloat162_rn(v);
    return *reinterpret_cast<const uint32_t*>(&h);
}
// Tells the compiler that the packed values may have changed, at no cost in instructions: without it, it keeps the
// unpacked fp32 form of all kept values alive from one pass over them to the next (twice the registers, spilled).
template <int N>
__device__ __forceinline__ void forget_unpacked(uint32_t (&h)[N]) {
#pragma unroll
    for (int i = 0; i < N; ++i) asm volatile("" : "+r"(h[i]));
}
__device__ __forceinline__ float2 unpack_bf16x2(uint32_t w) {
    return make_float2(__uint_as_float(w << 16), __uint_as_float(w & 0xFFFF0000u));
}
__device__ __forceinline__ uint4 ldg_u4(const void* p) { return __ldg(reinterpret_cast<const uint4*>(p)); }
__device__ __forceinline__ uint2 ldg_u2(const void* p) {
    uint2 v;
    asm volatile("ld.global.nc.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}
// a + b of two packed bf16 pairs, each sum rounded to bf16 (what a tensor addition stores)
__device__ __forceinline__ uint32_t add_bf16x2(uint32_t a, uint32_t b) {
    const __nv_bfloat162 r = __hadd2_rn(*reinterpret_cast<const __nv_bfloat162*>(&a), *reinterpret_cast<const __nv_bfloat162*>(&b));
    return *reinterpret_cast<const uint32_t*>(&r);
}
__device__ __forceinline__ float4 ldg_f4(const void* p) { return __ldg(reinterpret_cast<const float4*>(p)); }

template <int N_COLS>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(kThreads, 1)
token_project_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_o,
                     const __grid_constant__ TPArgs g) {
    constexpr int NC = N_COLS / 2;               // columns of this CTA: the pair splits the model width
    constexpr int CPT = NC / 4;                  // columns per thread
    constexpr int NP = CPT / 2;                  // packed bf16 pairs it holds
    constexpr uint32_t kWKBlockBytes = NC * 128; // this CTA's W rows of one K block
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint64_t full_bar[kAStages];      // gathered A tile has landed (one arrival per thread)
    __shared__ uint64_t w_full;                  // this CTA's rows of W are resident
    __shared__ uint64_t tmem_full[2];            // accumulator buffer complete (tcgen05.commit)
    __shared__ uint64_t tmem_free[2];            // every warp has read its columns of the buffer
    // Per lane quarter, one barrier for each of the two exchanges of a tile: the eight warps (four here, four in the
    // other CTA) that share its rows have written their partial statistics.  Two barriers, not one with alternating
    // phases: a warp of the other CTA may arrive for the next exchange while an arrival for this one is still on its
    // way, and on a single barrier that early arrival would be counted for the wrong phase.
    __shared__ uint64_t ex_bar[4][2];
    __shared__ uint32_t tmem_base_slot;

    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t* w_s = smem;                                               // [k_blocks][NC rows][128 B]
    uint8_t* a_s = w_s + kMaxKBlocks * kWKBlockBytes;                  // [stages][k_blocks][128 rows][128 B]
    uint8_t* box_s = a_s + kAStages * kAStageBytes;                    // [16 warps][32 rows][128 B]
    float2* ex1 = reinterpret_cast<float2*>(box_s + kWarps * kBoxBytes);      // [8][128] (local mean, local M2) of the 8 column groups
    float* ex2 = reinterpret_cast<float*>(ex1 + 8 * kRows);            // [8][128] partial sums of squares
    float* pvec = ex2 + 8 * kRows;                                     // [4][NC] fp32: bias, ln gamma, ln beta, rms gamma of this CTA's columns
    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = cluster_rank();       // which half of the columns
    const int32_t pair = static_cast<int32_t>(blockIdx.x >> 1);
    const int32_t n_pairs = static_cast<int32_t>(gridDim.x >> 1);
    const int32_t n_rows = static_cast<int32_t>(g.rows);
    const int32_t tiles = (n_rows + kRows - 1) / kRows;
    const int k_blocks = g.k_blocks;
    const int32_t my_tiles = pair < tiles ? (tiles - pair + n_pairs - 1) / n_pairs : 0;   // tiles this pair walks

    if (threadIdx.x == 0) {
        for (int s = 0; s < 2; ++s) {
            mbar_init(&full_bar[s], kThreads);
            mbar_init(&tmem_full[s], 1);
            mbar_init(&tmem_free[s], kWarps);
        }
        mbar_init(&w_full, 1);
        for (int q = 0; q < 4; ++q) {
            mbar_init(&ex_bar[q][0], 8);
            mbar_init(&ex_bar[q][1], 8);
        }
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(&tmem_base_slot, 2 * NC);
        tmem_relinquish();
    }
    for (int i = threadIdx.x; i < NC; i += kThreads) {
        const int col = static_cast<int>(cluster_rank()) * NC + i;
        pvec[i] = g.bias != nullptr ? g.bias[col] : 0.f;
        pvec[NC + i] = __bfloat162float(g.ln_gamma[col]);
        pvec[2 * NC + i] = __bfloat162float(g.ln_beta[col]);
        pvec[3 * NC + i] = __bfloat162float(g.rms_gamma[col]);
    }
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                          // the peer's shared memory exists before anything is written into it
    tc_fence_after_sync();
    const uint32_t tmem_base = tmem_base_slot;

    // W: rows [NC rank, NC rank + NC) of the weight, one box per K block, resident for the kernel's life
    if (threadIdx.x == 0) {
        tma_prefetch_desc(&tmap_w);
        mbar_expect_tx(&w_full, static_cast<uint32_t>(k_blocks) * kWKBlockBytes);
        for (int kb = 0; kb < k_blocks; ++kb)
            tma_load_3d(w_s + kb * kWKBlockBytes, &tmap_w, kb * 128, static_cast<int>(rank) * NC, 0, &w_full);
    }

    // ---- gather of one 128-row A tile: warp w copies rows [8 w, 8 w + 8); emb / 8 lanes copy one feature row.
    // Both CTAs of the pair gather the same rows (the second read of a table row is served by the L2).
    // Every thread makes K / 32 copies per tile (at most four).  Their table-row ids are read one tile before the copies
    // are issued (`load_ids`), so that the copies never wait for an id to arrive from HBM.
    uint32_t gid[4];
    auto load_ids = [&](int32_t it_local) {
        uint32_t tid_v;
        asm volatile("mov.u32 %0, %%tid.x;" : "=r"(tid_v));
        const int gw = static_cast<int>(tid_v >> 5), gl = static_cast<int>(tid_v & 31);
        const int chunks_f = g.emb >> 3;                  // 16-byte pieces of one feature's row: 4, 8 or 16
        const int per_feat = chunks_f >> 2;               // copies per thread and feature: 8 rows / (32 / chunks_f)
        const int sub_row = gl / chunks_f;
        const int32_t row0 = (pair + it_local * n_pairs) * kRows;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int f = q / per_feat;
            const int i = (q - f * per_feat) * (32 / chunks_f);
            uint32_t id = 0;
            if (f < g.n_feat && g.table[f] != nullptr) {
                const int64_t r = min(row0 + gw * 8 + i + sub_row, n_rows - 1);
                const int64_t v = g.ids[static_cast<int64_t>(f) * g.rows + r];
                id = static_cast<uint32_t>(min(max(v, static_cast<int64_t>(0)), g.table_rows[f] - 1));
            }
            gid[q] = id;
        }
    };
    auto gather = [&](int32_t it_local) {
        // thread and layout constants are derived afresh from a volatile read of the thread id on every call: kept
        // alive across the epilogue they would cost a dozen registers
        uint32_t tid_v;
        asm volatile("mov.u32 %0, %%tid.x;" : "=r"(tid_v));
        const int gw = static_cast<int>(tid_v >> 5), gl = static_cast<int>(tid_v & 31);
        const int chunks_f = g.emb >> 3;
        const int per_feat = chunks_f >> 2;
        const int sub_row = gl / chunks_f;
        const int piece = gl - sub_row * chunks_f;
        const uint32_t stage = smem_u32(a_s) + (static_cast<uint32_t>(it_local) & 1u) * kAStageBytes;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int f = q / per_feat;
            if (f < g.n_feat) {
                const int tile_row = gw * 8 + (q - f * per_feat) * (32 / chunks_f) + sub_row;
                const int col_piece = f * chunks_f + piece;          // 16-byte piece inside the K-wide row
                const uint32_t dst = stage + (col_piece >> 3) * kKBlockBytes + tile_row * 128 + (((col_piece & 7) ^ (tile_row & 7)) << 4);
                const __nv_bfloat16* table = g.table[f];
                const __nv_bfloat16* src = table != nullptr ? table + static_cast<int64_t>(gid[q]) * g.emb + piece * 8 : g.table_a;
                cp_async16(dst, src, table != nullptr ? 16u : 0u);
            }
        }
    };
    // ---- MMAs of one tile into accumulator buffer it & 1, issued by one thread
    auto issue = [&](int32_t it_local) -> bool {
        const uint32_t b = static_cast<uint32_t>(it_local) & 1u;
        const uint32_t use = static_cast<uint32_t>(it_local >> 1) & 1u;
        if (it_local == 0 && !mbar_wait_sleep(&w_full, 0)) return false;
        if (!mbar_wait_sleep(&tmem_free[b], use ^ 1u) || !mbar_wait_sleep(&full_bar[b], use)) return false;
        tc_fence_after_sync();
        const uint32_t idesc = umma_idesc(1, 1, 0, 0, kRows, NC);
        const uint64_t desc0 = umma_desc_sw128(0, 1024, 16);
        const uint32_t a_lo = (smem_u32(a_s) & 0x3FFFFu) >> 4;
        const uint32_t w_lo = (smem_u32(w_s) & 0x3FFFFu) >> 4;
        for (int kb = 0; kb < k_blocks; ++kb) {
            const uint64_t da = desc0 + a_lo + ((b * kAStageBytes + kb * kKBlockBytes) >> 4);
            const uint64_t db = desc0 + w_lo + ((kb * kWKBlockBytes) >> 4);
#pragma unroll
            for (int k = 0; k < 4; ++k) mma_f16_ss(tmem_base + b * NC, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
        }
        tc_commit(&tmem_full[b]);
        return true;
    };

    const int quarter = warp & 3;             // TMEM lanes [32 quarter, +32) are the ones this warp may read
    const int cg = warp >> 2;                 // which quarter of this CTA's columns
    const int col0 = static_cast<int>(rank) * NC + cg * CPT;     // first of this thread's columns in the full row
    const int row_in_tile = quarter * 32 + lane;
    uint8_t* box = box_s + warp * kBoxBytes;
    const int swz = lane & 7;
    const int slot = (static_cast<int>(rank) * 4 + cg) * kRows + row_in_tile;   // this thread's place in the exchange tables
    const uint32_t ex1_peer = map_to_peer(smem_u32(ex1 + slot), rank ^ 1u);
    const uint32_t ex2_peer = map_to_peer(smem_u32(ex2 + slot), rank ^ 1u);
    const uint32_t exbar_peer = map_to_peer(smem_u32(&ex_bar[quarter][0]), rank ^ 1u);
    // The eight warps that hold parts of the same 32 rows meet at ex_bar[quarter] twice per tile: every warp writes its
    // partials here and into the other CTA, then one lane arrives on both CTAs' barriers (release at cluster scope,
    // after the warp's writes) and the warp waits on its own CTA's.  Warps of other row quarters are not involved, so
    // the quarters drift apart and fill each other's stalls.
    auto exchange_arrive = [&](int which) {      // which: 0 = LayerNorm sums, 1 = RMS sum of the tile
        __syncwarp();                            // the warp's partial writes come before its one arrival
        if (lane == 0) {
            asm volatile("mbarrier.arrive.release.cluster.shared::cta.b64 _, [%0];" ::"r"(smem_u32(&ex_bar[quarter][which])) : "memory");
            asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(exbar_peer + 8u * which) : "memory");
        }
    };
    auto exchange_wait = [&](int which, uint32_t tile) -> bool {    // every lane waits (and so acquires the other warps' writes) itself
        return __all_sync(0xffffffffu, wait_cluster(&ex_bar[quarter][which], tile & 1u, kWait) ? 1 : 0) != 0;
    };
    constexpr float kInvN = 1.0f / N_COLS;
    bool ok = true;

    // ---- prologue: tiles 0 and 1 on their way, tile 0 signalled, its MMAs issued
    load_ids(0);
    if (my_tiles > 0) gather(0);
    asm volatile("cp.async.commit_group;" ::: "memory");
    load_ids(1);
    if (my_tiles > 1) gather(1);
    asm volatile("cp.async.commit_group;" ::: "memory");
    load_ids(2);
    asm volatile("cp.async.wait_group 1;" ::: "memory");
    fence_proxy_async_smem();                 // the copied rows are visible to the tensor core's proxy before the signal
    mbar_arrive(&full_bar[0]);
    if (warp == 0 && my_tiles > 0) {
        int passed = 1;
        if (lane == 0) passed = issue(0) ? 1 : 0;
        if (__shfl_sync(0xffffffffu, passed, 0) == 0) ok = false;
    }

    for (int32_t it = 0; it < my_tiles; ++it) {
        const int32_t m0 = (pair + it * n_pairs) * kRows;
        const uint32_t b = static_cast<uint32_t>(it) & 1u;
        // ---- the next tile's rows have landed (copies issued a tile ago): signal
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (it + 1 < my_tiles) {
            fence_proxy_async_smem();
            mbar_arrive(&full_bar[b ^ 1u]);
        }
        // A warp whose wait gives up stops waiting but keeps walking the tiles, so that it still meets every barrier
        // and every arrival the others count on; its output is garbage and the status word says so.
        if (ok) {   // one lane polls, the warp follows
            int passed = 1;
            if (lane == 0) passed = mbar_wait_sleep(&tmem_full[b], static_cast<uint32_t>(it >> 1) & 1u) ? 1 : 0;
            if (__shfl_sync(0xffffffffu, passed, 0) == 0) ok = false;
        }
        tc_fence_after_sync();
        // the MMAs of this tile are done: its A stage is free for the tile after the next
        if (it + 2 < my_tiles) gather(it + 2);
        asm volatile("cp.async.commit_group;" ::: "memory");
        load_ids(it + 3);                        // rows past the end are clamped: the ids are simply not used

        const int32_t row = min(m0 + row_in_tile, n_rows - 1);   // rows past the end repeat the last one (nothing of theirs is stored)
        const bool row_ok = m0 + row_in_tile < n_rows;
        const int32_t id_a = static_cast<int32_t>(min(max(g.ids_a[row], static_cast<int64_t>(0)), g.rows_a - 1));
        const int32_t id_b = g.table_b != nullptr ? static_cast<int32_t>(min(max(g.ids_b[row], static_cast<int64_t>(0)), g.rows_b - 1)) : 0;
        int32_t dst_row = g.row_dst != nullptr ? g.row_dst[row] : row;
        if (!row_ok || dst_row >= g.rows_out) dst_row = -1;
        const __nv_bfloat16* ta = g.table_a + static_cast<int64_t>(id_a) * N_COLS + col0;
        const __nv_bfloat16* tb = g.table_b != nullptr ? g.table_b + static_cast<int64_t>(id_b) * N_COLS + col0 : nullptr;
        asm volatile("prefetch.global.L1 [%0];" ::"l"(ta));      // this thread's 2 * CPT bytes of the two rows: one line each
        if (tb != nullptr) asm volatile("prefetch.global.L1 [%0];" ::"l"(tb));

        // ---- pass 1: accumulator columns -> bf16 SiLU values in registers
        const uint32_t taddr = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + b * NC + cg * CPT;
        uint32_t h[NP];
        float2 s1 = make_float2(0.f, 0.f), s2 = make_float2(0.f, 0.f);     // sum and sum of squares of the SiLU values
        {
            uint32_t acc[CPT / 16][16];
#pragma unroll
            for (int c = 0; c < CPT / 16; ++c) tmem_ld_x16(taddr + 16 * c, acc[c]);     // back to back, one wait
#pragma unroll
            for (int c = 0; c < CPT / 16; ++c) tc_wait_ld(acc[c]);                      // (the first one waits for all of them)
            const float* bias_s = pvec + cg * CPT;
#pragma unroll
            for (int c = 0; c < CPT / 16; ++c) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float4 bv = *reinterpret_cast<const float4*>(bias_s + 16 * c + 4 * j);
                    const float2 v0 = silu2(__fadd2_rn(make_float2(__uint_as_float(acc[c][4 * j]), __uint_as_float(acc[c][4 * j + 1])), make_float2(bv.x, bv.y)));
                    const float2 v1 = silu2(__fadd2_rn(make_float2(__uint_as_float(acc[c][4 * j + 2]), __uint_as_float(acc[c][4 * j + 3])), make_float2(bv.z, bv.w)));
                    s1 = __fadd2_rn(s1, __fadd2_rn(v0, v1));
                    s2 = __ffma2_rn(v0, v0, s2);
                    s2 = __ffma2_rn(v1, v1, s2);
                    h[8 * c + 2 * j] = pack_bf16x2(v0);
                    h[8 * c + 2 * j + 1] = pack_bf16x2(v1);
                }
            }
        }
        tc_fence_before_sync();
        __syncwarp();
        if (lane == 0) mbar_arrive(&tmem_free[b]);   // the MMAs of the tile after the next may overwrite this buffer
        // the next tile's MMAs go into the other buffer and run under the rest of this epilogue; by now every warp has
        // signalled that tile's rows, so the issuing warp does not wait for stragglers
        if (warp == 0 && it + 1 < my_tiles) {
            int passed = 1;
            if (lane == 0 && ok) passed = issue(it + 1) ? 1 : 0;
            if (__shfl_sync(0xffffffffu, passed, 0) == 0) ok = false;
        }

        // ---- LayerNorm statistics: this thread's sum and sum of squares (fp32, taken in pass 1) meet those of the
        // row's other seven column groups, four of them in the other CTA
        ex1[slot] = make_float2(s1.x + s1.y, s2.x + s2.y);
        st_cluster_f2(ex1_peer, s1.x + s1.y, s2.x + s2.y);
        exchange_arrive(0);
        if (!exchange_wait(0, static_cast<uint32_t>(it)) && ok) ok = false;
        float mean = 0.f, m2 = 0.f;
#pragma unroll
        for (int q = 0; q < 8; ++q) {
            const float2 part = ex1[q * kRows + row_in_tile];
            mean += part.x;
            m2 += part.y;
        }
        mean *= kInvN;
        const float rstd1 = rsqrtf(fmaxf(fmaf(-mean, mean, m2 * kInvN), 0.f) + g.ln_eps);
        const float2 nmean = make_float2(-mean, -mean);
        const float2 rstd = make_float2(rstd1, rstd1);

        // ---- normalise, add the table rows (one rounding per sum, like tensor additions), RMS partial sum
        float2 acc2 = make_float2(0.f, 0.f);
        const float* gam_s = pvec + NC + cg * CPT;
        const float* bet_s = pvec + 2 * NC + cg * CPT;
#pragma unroll
        for (int c = 0; c < CPT / 8; ++c) {
            const uint4 aw = ldg_u4(ta + 8 * c);
            const uint32_t aws[4] = {aw.x, aw.y, aw.z, aw.w};
            uint32_t w[4];
#pragma unroll
            for (int e = 0; e < 4; e += 2) {
                const float4 g4 = *reinterpret_cast<const float4*>(gam_s + 8 * c + 2 * e);
                const float4 b4 = *reinterpret_cast<const float4*>(bet_s + 8 * c + 2 * e);
                w[e] = pack_bf16x2(__ffma2_rn(__fmul2_rn(__fadd2_rn(unpack_bf16x2(h[4 * c + e]), nmean), rstd), make_float2(g4.x, g4.y), make_float2(b4.x, b4.y)));
                w[e + 1] = pack_bf16x2(__ffma2_rn(__fmul2_rn(__fadd2_rn(unpack_bf16x2(h[4 * c + e + 1]), nmean), rstd), make_float2(g4.z, g4.w), make_float2(b4.z, b4.w)));
                w[e] = add_bf16x2(w[e], aws[e]);
                w[e + 1] = add_bf16x2(w[e + 1], aws[e + 1]);
            }
            if (tb != nullptr) {
                const uint4 b2 = ldg_u4(tb + 8 * c);
                w[0] = add_bf16x2(w[0], b2.x);
                w[1] = add_bf16x2(w[1], b2.y);
                w[2] = add_bf16x2(w[2], b2.z);
                w[3] = add_bf16x2(w[3], b2.w);
            }
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                h[4 * c + e] = w[e];
                const float2 tv = unpack_bf16x2(w[e]);
                acc2 = __ffma2_rn(tv, tv, acc2);
            }
        }
        forget_unpacked(h);
        ex2[slot] = acc2.x + acc2.y;
        st_cluster_f1(ex2_peer, acc2.x + acc2.y);
        exchange_arrive(1);
        if (!exchange_wait(1, static_cast<uint32_t>(it)) && ok) ok = false;
        float sq = 0.f;
#pragma unroll
        for (int q = 0; q < 8; ++q) sq += ex2[q * kRows + row_in_tile];
        const float rms1 = rsqrtf(sq * kInvN + g.rms_eps);
        const float2 rms = make_float2(rms1, rms1);

        // ---- `tokens`: only rows that a destination was given for
        if (dst_row >= 0) {
            uint4* out = reinterpret_cast<uint4*>(g.tokens + static_cast<int64_t>(dst_row) * N_COLS + col0);
#pragma unroll
            for (int c = 0; c < CPT / 8; ++c) out[c] = make_uint4(h[4 * c], h[4 * c + 1], h[4 * c + 2], h[4 * c + 3]);
        }

        // ---- `normed`: the warp's 32 rows x CPT columns through its staging box (128-byte rows at CPT = 64)
        if (lane == 0) bulk_wait_read<0>();     // this warp's previous store has read the box
        __syncwarp();
        const float* rg_s = pvec + 3 * NC + cg * CPT;
#pragma unroll
        for (int c = 0; c < CPT / 8; ++c) {
            const float4 g0 = *reinterpret_cast<const float4*>(rg_s + 8 * c);
            const float4 g1 = *reinterpret_cast<const float4*>(rg_s + 8 * c + 4);
            uint4 o;
            o.x = pack_bf16x2(__fmul2_rn(__fmul2_rn(unpack_bf16x2(h[4 * c]), rms), make_float2(g0.x, g0.y)));
            o.y = pack_bf16x2(__fmul2_rn(__fmul2_rn(unpack_bf16x2(h[4 * c + 1]), rms), make_float2(g0.z, g0.w)));
            o.z = pack_bf16x2(__fmul2_rn(__fmul2_rn(unpack_bf16x2(h[4 * c + 2]), rms), make_float2(g1.x, g1.y)));
            o.w = pack_bf16x2(__fmul2_rn(__fmul2_rn(unpack_bf16x2(h[4 * c + 3]), rms), make_float2(g1.z, g1.w)));
            // CPT = 64: eight 16-byte pieces per row, 128-byte swizzle; CPT = 32: four pieces, 64-byte swizzle
            const int pc = CPT == 64 ? (c ^ swz) : (c ^ ((lane >> 1) & 3));
            *reinterpret_cast<uint4*>(box + lane * (2 * CPT) + (pc << 4)) = o;
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
            const int32_t y0 = m0 + quarter * 32;
            if (y0 < n_rows) tma_store_3d(&tmap_o, box, 2 * col0, y0, 0);   // rows past the end are clipped
            bulk_commit();
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    if (lane == 0) bulk_wait<0>();            // the last store must have left shared memory before the CTA ends
    if (!ok && g.status != nullptr) atomicExch(g.status, 1);

    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();                          // the peer may still write this CTA's exchange tables
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, 2 * NC);
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

// [1, rows, row_bytes] bytes, boxes of box_rows x box_bytes (128 or 64), swizzle of the box width
bool make_tmap(CUtensorMap* map, const void* base, uint64_t row_bytes, uint64_t rows, uint32_t box_rows, uint32_t box_bytes) {
    PFN_cuTensorMapEncodeTiled_v12000 fn = encode_fn();
    if (fn == nullptr) return false;
    const cuuint64_t dims[3] = {row_bytes, rows, 1};
    const cuuint64_t strides[2] = {row_bytes, row_bytes * rows};
    const cuuint32_t box[3] = {box_bytes, box_rows, 1};
    const cuuint32_t elem[3] = {1, 1, 1};
    const CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, elem,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, box_bytes == 64 ? CU_TENSOR_MAP_SWIZZLE_64B : CU_TENSOR_MAP_SWIZZLE_128B,
                          CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS;
}

template <int N_COLS>
int launch(const CUtensorMap& tw, const CUtensorMap& to, const TPArgs& g, cudaStream_t stream) {
    constexpr size_t smem = kMaxKBlocks * (N_COLS / 2) * 128 + kAStages * kAStageBytes + kWarps * kBoxBytes +
                            8 * kRows * sizeof(float2) + 8 * kRows * sizeof(float) + 4 * (N_COLS / 2) * sizeof(float) + 1024;
    const DeviceInfo& dev = device_info();
    static bool attr_set[64] = {};
    if (!attr_set[dev.index]) {
        cudaFuncSetAttribute(token_project_kernel<N_COLS>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem));
        attr_set[dev.index] = true;
    }
    const int64_t tiles = (g.rows + kRows - 1) / kRows;
    int64_t pairs = dev.sm_count / 2;
    if (pairs > tiles) pairs = tiles;
    token_project_kernel<N_COLS><<<static_cast<unsigned>(2 * pairs), kThreads, smem, stream>>>(tw, to, g);
    count_launch();
    return launch_status();
}

}  // namespace
}  // namespace tb200

extern "C" int tb200_token_project_fwd(const void* const* tables, const int64_t* table_rows, int32_t n_feat, int32_t emb,
                                       const int64_t* ids, const void* w, const float* bias, const void* ln_gamma,
                                       const void* ln_beta, const void* table_a, int64_t rows_a, const int64_t* ids_a,
                                       const void* table_b, int64_t rows_b, const int64_t* ids_b, const void* rms_gamma,
                                       const int32_t* row_dst, int64_t rows_out, void* tokens, void* normed, int64_t rows,
                                       int32_t n_cols, float ln_eps, float rms_eps, int32_t* status_word, void* stream) {
    using namespace tb200;
    if (rows < 0 || rows_out < 0 || n_feat < 1 || n_feat > kMaxFeat || rows_a < 1 || (table_b != nullptr && rows_b < 1))
        return TB200_ERR_SHAPE;
    if (n_cols != 256 && n_cols != 512) return TB200_ERR_UNSUPPORTED;
    // a feature's row is emb / 8 sixteen-byte pieces copied by as many lanes, and a warp copies eight rows of a tile:
    // 4, 8 or 16 lanes per row; K = n_feat * emb = 64 or 128
    if (emb != 32 && emb != 64 && emb != 128) return TB200_ERR_UNSUPPORTED;
    const int64_t k = static_cast<int64_t>(n_feat) * emb;
    if (k != 64 && k != 128) return TB200_ERR_UNSUPPORTED;
    if (rows == 0) return TB200_OK;
    if (rows > 0x7FF00000ll || rows_a > 0x7FFFFFFFll || rows_b > 0x7FFFFFFFll) return TB200_ERR_SHAPE;   // 32-bit row arithmetic, with room for the ids read three tiles ahead
    if (tables == nullptr || table_rows == nullptr || ids == nullptr || w == nullptr || ln_gamma == nullptr ||
        ln_beta == nullptr || table_a == nullptr || ids_a == nullptr || rms_gamma == nullptr || tokens == nullptr ||
        normed == nullptr || (table_b != nullptr && ids_b == nullptr))
        return TB200_ERR_NULL;
    TPArgs g{};
    for (int f = 0; f < n_feat; ++f) {
        if (tables[f] != nullptr && (table_rows[f] < 1 || !aligned16(tables[f]))) return tables[f] != nullptr && table_rows[f] < 1 ? TB200_ERR_SHAPE : TB200_ERR_ALIGN;
        g.table[f] = static_cast<const __nv_bfloat16*>(tables[f]);
        g.table_rows[f] = tables[f] != nullptr ? table_rows[f] : 1;
    }
    if (!aligned16(w) || !aligned16(ln_gamma) || !aligned16(ln_beta) || !aligned16(rms_gamma) || !aligned16(table_a) ||
        (table_b != nullptr && !aligned16(table_b)) || !aligned16(tokens) || !aligned16(normed) ||
        (bias != nullptr && !aligned16(bias)))
        return TB200_ERR_ALIGN;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    CUtensorMap tw, to;
    if (!make_tmap(&tw, w, 2ull * k, static_cast<uint64_t>(n_cols), static_cast<uint32_t>(n_cols / 2), 128) ||
        !make_tmap(&to, normed, 2ull * n_cols, static_cast<uint64_t>(rows), 32, static_cast<uint32_t>(n_cols / 4)))
        return TB200_ERR_DRIVER;
    g.ids = ids;
    g.bias = bias;
    g.ln_gamma = static_cast<const __nv_bfloat16*>(ln_gamma);
    g.ln_beta = static_cast<const __nv_bfloat16*>(ln_beta);
    g.rms_gamma = static_cast<const __nv_bfloat16*>(rms_gamma);
    g.table_a = static_cast<const __nv_bfloat16*>(table_a);
    g.table_b = static_cast<const __nv_bfloat16*>(table_b);
    g.ids_a = ids_a;
    g.ids_b = ids_b;
    g.row_dst = row_dst;
    g.tokens = static_cast<__nv_bfloat16*>(tokens);
    g.status = status_word;
    g.rows = rows;
    g.rows_a = rows_a;
    g.rows_b = rows_b;
    g.rows_out = row_dst != nullptr ? rows_out : rows;
    g.n_feat = n_feat;
    g.emb = emb;
    g.k_blocks = static_cast<int32_t>(k / 64);
    g.ln_eps = ln_eps;
    g.rms_eps = rms_eps;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (n_cols == 512) return launch<512>(tw, to, g, s);
    return launch<256>(tw, to, g, s);
}
