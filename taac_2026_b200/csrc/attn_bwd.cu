// Attention backward for the padded (B, H, L, D) layout: dq, dk, dv from q, k, v, o and the upstream gradient, with
// the same mask rule as the forward kernels (valid prefix, always-valid suffix, causal, key-validity map, padded
// queries that return their own value row).  It is the first, plain form of the training-side kernel (the reference's
// is `flash_attention_backward`, accelerators/attention/kernels/tilelang.py:440-701): fp32 arithmetic on the CUDA
// cores, scores recomputed instead of stored, two kernels and no atomics, so the gradients do not depend on
// scheduling:
//   query kernel   one warp per (sample, head, query i):  scores -> row maximum and sum (their log2 "lse" and
//                  delta_i = dO_i . O_i go to a workspace), ds_ij = p_ij (dO_i . v_j - delta_i),
//                  dq_i = scale * sum_j ds_ij k_j
//   key kernel     one warp per (sample, head, key j):    p_ij = exp2(s_ij - lse_i) for the queries that see j,
//                  dv_j = sum_i p_ij dO_i,  dk_j = scale * sum_i ds_ij q_i
// A padded query (forward: o_i = v_i) passes its gradient straight to dv_i and has no dq; a query without a visible
// key (forward: zeros) has no gradient at all.  Work is O(Lq Lk D) per kernel without tensor cores: meant for
// correctness and for small training shapes, not for the serving path.
#include <cuda_bf16.h>
#include <cuda_fp16.h>

#include "attn_common.cuh"
#include "tb200_common.cuh"

namespace tb200 {
void count_launch();

namespace {

constexpr int kMaxD = 256;
constexpr int kMaxL = 4096;
constexpr float kSelfRow = INFINITY;      // lse marker: padded query, gradient goes to its own value row
constexpr float kEmptyRow = -INFINITY;    // lse marker: no visible key

struct BwdArgs {
    AttnArgs a;                 // q, k, v, o and their strides, the mask
    const void* d_o;            // strides of o
    void* dq;                   // strides of q
    void* dk;                   // strides of k
    void* dv;                   // strides of v
    float* lse;                 // [B, H, Lq]
    float* delta;               // [B, H, Lq]
    float scale;
};

template <typename T>
__device__ __forceinline__ float to_f(T x) { return static_cast<float>(x); }
template <>
__device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 x) { return __bfloat162float(x); }
template <>
__device__ __forceinline__ float to_f<__half>(__half x) { return __half2float(x); }
template <typename T>
__device__ __forceinline__ T from_f(float x) { return static_cast<T>(x); }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }
template <>
__device__ __forceinline__ __half from_f<__half>(float x) { return __float2half_rn(x); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

struct RowMask {
    int valid_len, ns_start, lk;
    bool causal;
    const uint8_t* kvalid;
    __device__ __forceinline__ bool sees(int query, int key) const {
        return kvalid != nullptr ? (kvalid[key] != 0 && (!causal || key <= query))
                                 : attn_visible(query, key, valid_len, ns_start, lk, causal);
    }
    __device__ __forceinline__ bool padded_query(int pos) const {
        return kvalid != nullptr ? kvalid[pos] == 0 : (pos >= valid_len && pos < ns_start);
    }
};

__device__ __forceinline__ RowMask make_mask(const AttnArgs& a, int b) {
    RowMask m;
    m.lk = a.Lk;
    m.valid_len = a.seq_len != nullptr ? min(max(a.seq_len[b], 0), a.Lk) : a.Lk;
    m.ns_start = min(a.ns_start, a.Lk);
    m.causal = a.causal != 0;
    m.kvalid = a.key_valid != nullptr ? a.key_valid + static_cast<int64_t>(b) * a.Lk : nullptr;
    return m;
}

constexpr int kWarpsQ = 4;

template <typename T>
__global__ void __launch_bounds__(kWarpsQ * 32)
attn_bwd_query_kernel(const BwdArgs g, const int D) {
    extern __shared__ float smem[];
    const AttnArgs& a = g.a;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* qs = smem + warp * (2 * kMaxD + a.Lk);      // q_i, dO_i, then one value per key
    float* gs = qs + kMaxD;
    float* ps = gs + kMaxD;
    const int b = blockIdx.x, h = blockIdx.y;
    const int i = blockIdx.z * kWarpsQ + warp;
    if (i >= a.Lq) return;                              // whole warps leave: no block-wide barrier below
    const RowMask mask = make_mask(a, b);
    const int64_t row = (static_cast<int64_t>(b) * a.H + h) * a.Lq + i;
    const T* qp = static_cast<const T*>(a.q) + b * a.q_sb + h * a.q_sh + static_cast<int64_t>(i) * a.q_sl;
    const T* op = static_cast<const T*>(a.o) + b * a.o_sb + h * a.o_sh + static_cast<int64_t>(i) * a.o_sl;
    const T* gp = static_cast<const T*>(g.d_o) + b * a.o_sb + h * a.o_sh + static_cast<int64_t>(i) * a.o_sl;
    const T* kp = static_cast<const T*>(a.k) + b * a.k_sb + h * a.k_sh;
    const T* vp = static_cast<const T*>(a.v) + b * a.v_sb + h * a.v_sh;
    T* dqp = static_cast<T*>(g.dq) + b * a.q_sb + h * a.q_sh + static_cast<int64_t>(i) * a.q_sl;

    if (a.padded_query_self && i < a.Lk && mask.padded_query(i)) {
        for (int d = lane; d < D; d += 32) dqp[d] = from_f<T>(0.f);
        if (lane == 0) { g.lse[row] = kSelfRow; g.delta[row] = 0.f; }
        return;
    }
    float part = 0.f;
    for (int d = lane; d < D; d += 32) {
        qs[d] = to_f(qp[d]);
        gs[d] = to_f(gp[d]);
        part += gs[d] * to_f(op[d]);
    }
    const float delta = warp_sum(part);
    __syncwarp();
    // pass 1: one key per lane, scores in the log2 domain
    float row_max = -INFINITY;
    for (int j = lane; j < a.Lk; j += 32) {
        float s = -INFINITY;
        if (mask.sees(i, j)) {
            const T* kr = kp + static_cast<int64_t>(j) * a.k_sl;
            float dot = 0.f;
            for (int d = 0; d < D; ++d) dot = fmaf(qs[d], to_f(kr[d]), dot);
            s = dot * a.scale_log2;
        }
        ps[j] = s;
        row_max = fmaxf(row_max, s);
    }
    row_max = warp_max(row_max);
    if (row_max == -INFINITY) {                         // no visible key: the forward wrote zeros
        for (int d = lane; d < D; d += 32) dqp[d] = from_f<T>(0.f);
        if (lane == 0) { g.lse[row] = kEmptyRow; g.delta[row] = 0.f; }
        return;
    }
    float sum = 0.f;
    for (int j = lane; j < a.Lk; j += 32) sum += exp2f(ps[j] - row_max);
    sum = warp_sum(sum);
    const float lse = row_max + log2f(sum);
    if (lane == 0) { g.lse[row] = lse; g.delta[row] = delta; }
    // pass 2: ds_j = p_j (dO . v_j - delta), one key per lane
    for (int j = lane; j < a.Lk; j += 32) {
        float ds = 0.f;
        if (ps[j] != -INFINITY) {
            const T* vr = vp + static_cast<int64_t>(j) * a.v_sl;
            float dp = 0.f;
            for (int d = 0; d < D; ++d) dp = fmaf(gs[d], to_f(vr[d]), dp);
            ds = exp2f(ps[j] - lse) * (dp - delta);
        }
        ps[j] = ds;
    }
    __syncwarp();
    // pass 3: dq_d = scale * sum_j ds_j k_jd, one output dimension per lane (coalesced key rows)
    const int last = mask.causal ? min(a.Lk, i + 1) : a.Lk;
    for (int d = lane; d < D; d += 32) {
        float acc = 0.f;
        for (int j = 0; j < last; ++j) acc = fmaf(ps[j], to_f(kp[static_cast<int64_t>(j) * a.k_sl + d]), acc);
        dqp[d] = from_f<T>(acc * g.scale);
    }
}

constexpr int kWarpsK = 2;

template <typename T>
__global__ void __launch_bounds__(kWarpsK * 32)
attn_bwd_key_kernel(const BwdArgs g, const int D) {
    extern __shared__ float smem[];
    const AttnArgs& a = g.a;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    float* ks = smem + warp * (2 * kMaxD + 2 * a.Lq);  // k_j, v_j, then p_i and ds_i per query
    float* vs = ks + kMaxD;
    float* ps = vs + kMaxD;
    float* ds = ps + a.Lq;
    const int b = blockIdx.x, h = blockIdx.y;
    const int j = blockIdx.z * kWarpsK + warp;
    if (j >= a.Lk) return;
    const RowMask mask = make_mask(a, b);
    const T* kr = static_cast<const T*>(a.k) + b * a.k_sb + h * a.k_sh + static_cast<int64_t>(j) * a.k_sl;
    const T* vr = static_cast<const T*>(a.v) + b * a.v_sb + h * a.v_sh + static_cast<int64_t>(j) * a.v_sl;
    const T* qp = static_cast<const T*>(a.q) + b * a.q_sb + h * a.q_sh;
    const T* gp = static_cast<const T*>(g.d_o) + b * a.o_sb + h * a.o_sh;
    T* dkp = static_cast<T*>(g.dk) + b * a.k_sb + h * a.k_sh + static_cast<int64_t>(j) * a.k_sl;
    T* dvp = static_cast<T*>(g.dv) + b * a.v_sb + h * a.v_sh + static_cast<int64_t>(j) * a.v_sl;
    const float* lse = g.lse + (static_cast<int64_t>(b) * a.H + h) * a.Lq;
    const float* delta = g.delta + (static_cast<int64_t>(b) * a.H + h) * a.Lq;
    for (int d = lane; d < D; d += 32) {
        ks[d] = to_f(kr[d]);
        vs[d] = to_f(vr[d]);
    }
    __syncwarp();
    const int first = mask.causal ? j : 0;              // with the causal rule only queries i >= j see key j
    for (int i = first + lane; i < a.Lq; i += 32) {
        float p = 0.f, dsv = 0.f;
        const float l = lse[i];
        if (l == kSelfRow) {
            p = i == j ? 1.f : 0.f;                     // o_i = v_i: the gradient of a padded query goes to its own row
        } else if (l != kEmptyRow && mask.sees(i, j)) {
            const T* qr = qp + static_cast<int64_t>(i) * a.q_sl;
            const T* gr = gp + static_cast<int64_t>(i) * a.o_sl;
            float dot = 0.f, dp = 0.f;
            for (int d = 0; d < D; ++d) {
                dot = fmaf(to_f(qr[d]), ks[d], dot);
                dp = fmaf(to_f(gr[d]), vs[d], dp);
            }
            p = exp2f(dot * a.scale_log2 - l);
            dsv = p * (dp - delta[i]);
        }
        ps[i] = p;
        ds[i] = dsv;
    }
    __syncwarp();
    for (int d = lane; d < D; d += 32) {
        float acc_v = 0.f, acc_k = 0.f;
        for (int i = first; i < a.Lq; ++i) {
            acc_v = fmaf(ps[i], to_f(gp[static_cast<int64_t>(i) * a.o_sl + d]), acc_v);
            acc_k = fmaf(ds[i], to_f(qp[static_cast<int64_t>(i) * a.q_sl + d]), acc_k);
        }
        dvp[d] = from_f<T>(acc_v);
        dkp[d] = from_f<T>(acc_k * g.scale);
    }
}

template <typename T>
int launch(const BwdArgs& g, int D, cudaStream_t stream) {
    const AttnArgs& a = g.a;
    const size_t smem_q = static_cast<size_t>(kWarpsQ) * (2 * kMaxD + a.Lk) * sizeof(float);
    const size_t smem_k = static_cast<size_t>(kWarpsK) * (2 * kMaxD + 2 * a.Lq) * sizeof(float);
    static bool attr_set[64] = {};
    const DeviceInfo& dev = device_info();
    if (!attr_set[dev.index]) {
        const int cap_q = static_cast<int>(kWarpsQ * (2 * kMaxD + kMaxL) * sizeof(float));
        const int cap_k = static_cast<int>(kWarpsK * (2 * kMaxD + 2 * kMaxL) * sizeof(float));
        cudaFuncSetAttribute(attn_bwd_query_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap_q);
        cudaFuncSetAttribute(attn_bwd_query_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap_q);
        cudaFuncSetAttribute(attn_bwd_query_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap_q);
        cudaFuncSetAttribute(attn_bwd_key_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap_k);
        cudaFuncSetAttribute(attn_bwd_key_kernel<__nv_bfloat16>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap_k);
        cudaFuncSetAttribute(attn_bwd_key_kernel<__half>, cudaFuncAttributeMaxDynamicSharedMemorySize, cap_k);
        attr_set[dev.index] = true;
    }
    const unsigned zq = static_cast<unsigned>((a.Lq + kWarpsQ - 1) / kWarpsQ);
    const unsigned zk = static_cast<unsigned>((a.Lk + kWarpsK - 1) / kWarpsK);
    attn_bwd_query_kernel<T><<<dim3(a.B, a.H, zq), kWarpsQ * 32, smem_q, stream>>>(g, D);
    count_launch();
    int code = launch_status();
    if (code != TB200_OK) return code;
    attn_bwd_key_kernel<T><<<dim3(a.B, a.H, zk), kWarpsK * 32, smem_k, stream>>>(g, D);
    count_launch();
    return launch_status();
}

}  // namespace
}  // namespace tb200

extern "C" int64_t tb200_attn_bwd_workspace_bytes(int32_t B, int32_t H, int32_t Lq) {
    if (B < 0 || H < 0 || Lq < 0) return 0;
    return static_cast<int64_t>(B) * H * Lq * 2 * static_cast<int64_t>(sizeof(float));
}

extern "C" int tb200_attn_bwd(const void* q, const void* k, const void* v, const void* o, const void* d_o, void* dq, void* dk,
                              void* dv, void* workspace, int32_t B, int32_t H, int32_t Lq, int32_t Lk, int32_t D,
                              const int64_t* strides, const int32_t* seq_len, const uint8_t* key_valid, int32_t ns_start,
                              int32_t causal, int32_t padded_query_self, float scale, int dtype, void* stream) {
    using namespace tb200;
    if (B < 0 || H < 1 || Lq < 0 || Lk < 0 || D < 1 || ns_start < 0) return TB200_ERR_SHAPE;
    if (B == 0 || Lq == 0 || Lk == 0) return TB200_OK;
    if (q == nullptr || k == nullptr || v == nullptr || o == nullptr || d_o == nullptr || dq == nullptr || dk == nullptr ||
        dv == nullptr || workspace == nullptr || strides == nullptr)
        return TB200_ERR_NULL;
    if (dtype != TB200_BF16 && dtype != TB200_F16 && dtype != TB200_F32) return TB200_ERR_DTYPE;
    if (D > kMaxD || Lq > kMaxL || Lk > kMaxL || H > 65535) return TB200_ERR_UNSUPPORTED;
    if (padded_query_self && Lq != Lk) return TB200_ERR_SHAPE;
    if (!device_info().valid) return TB200_ERR_DEVICE;
    BwdArgs g{};
    AttnArgs& a = g.a;
    a.q = q; a.k = k; a.v = v; a.o = const_cast<void*>(o);
    a.q_sb = strides[0]; a.q_sh = strides[1]; a.q_sl = strides[2];
    a.k_sb = strides[3]; a.k_sh = strides[4]; a.k_sl = strides[5];
    a.v_sb = strides[6]; a.v_sh = strides[7]; a.v_sl = strides[8];
    a.o_sb = strides[9]; a.o_sh = strides[10]; a.o_sl = strides[11];
    a.seq_len = seq_len;
    a.key_valid = key_valid;
    a.B = B; a.H = H; a.Lq = Lq; a.Lk = Lk;
    a.ns_start = ns_start > Lk ? Lk : ns_start;
    a.causal = causal != 0;
    a.padded_query_self = padded_query_self != 0;
    a.scale_log2 = scale * 1.4426950408889634f;
    g.d_o = d_o; g.dq = dq; g.dk = dk; g.dv = dv;
    g.lse = static_cast<float*>(workspace);
    g.delta = g.lse + static_cast<int64_t>(B) * H * Lq;
    g.scale = scale;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case TB200_F32: return launch<float>(g, D, s);
        case TB200_F16: return launch<__half>(g, D, s);
        default: return launch<__nv_bfloat16>(g, D, s);
    }
}
