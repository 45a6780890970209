// Router projection (scores = x W_r^T) and its backward, in fp32 semantics.
//
// Upstream runs the router under `set_matmul_precision(None)` (src/qutai/lm/layers.py:377-378): fp32
// weights, fp32 arithmetic, whatever the activation dtype.  Two implementations sit behind the same
// entry points:
//   * bf16 activations: the tensor cores, with every fp32 factor split into bf16 terms
//     (v = hi + mid + lo, 8 mantissa bits each, so hi + mid + lo carries all 24).  bf16 x bf16
//     products are exact in fp32 and the accumulation is fp32, so the result differs from an fp32
//     FMA chain only by fp32 rounding of the partial sums.  x itself is bf16 and needs no split.
//       scores      = x . (W_hi + W_mid + W_lo)^T                       one launch, K = d
//       dx_router   = ds . W_hi + (ds_hi + ds_mid) . W_mid              one launch, K = 6 S
//       dW_router   = (ds_hi + ds_mid + ds_lo)^T . x                    split over token blocks, reduced in a fixed order
//   * fp32 activations (or more than 64 experts): the CUDA-core GEMM of gemm_simt.cu.
#include "common.cuh"

namespace qmoe {
namespace {

constexpr long long kAlign = 256;
inline long long align_up(long long v) { return (v + kAlign - 1) / kAlign * kAlign; }

struct RouterScratch {  // byte offsets inside the caller's scratch buffer
    int S, splits;
    long long rows_per_split;
    long long w3, wbwd, ds6, tables, partial, total;
};

RouterScratch plan_scratch(long long T, int E, long long d) {
    RouterScratch r;
    r.S = (E + 31) / 32 * 32;
    long long splits = T / 1024;
    if (splits < 1) splits = 1;
    if (splits > 32) splits = 32;
    r.rows_per_split = ((T + splits - 1) / splits + kRowPad - 1) / kRowPad * kRowPad;
    r.splits = (int)((T + r.rows_per_split - 1) / r.rows_per_split);
    long long at = 0;
    r.w3 = at;      at = align_up(at + 3ll * r.S * d * 2);
    r.wbwd = at;    at = align_up(at + 6ll * r.S * d * 2);
    r.ds6 = at;     at = align_up(at + T * 6ll * r.S * 2);
    r.tables = at;  at = align_up(at + (2ll * r.splits + 1) * 4);
    r.partial = at; at = align_up(at + (long long)r.splits * 3 * r.S * d * 4);
    r.total = at;
    return r;
}

bool tc_router_ok(int x_dtype, int E, long long d, uint64_t x, uint64_t scratch) {
    return x_dtype == QMOE_BF16 && E <= 64 && d % 8 == 0 && d >= 64 && scratch && !(x & 15u) && !(scratch & 255u);
}

__device__ __forceinline__ void split3(float v, __nv_bfloat16& hi, __nv_bfloat16& mid, __nv_bfloat16& lo) {
    hi = __float2bfloat16_rn(v);
    const float r1 = v - __bfloat162float(hi);
    mid = __float2bfloat16_rn(r1);
    lo = __float2bfloat16_rn(r1 - __bfloat162float(mid));
}

// W [E, d] fp32 -> w3 [3S, d] = {hi; mid; lo}, wbwd [6S, d] = {hi; hi; hi; mid; mid; 0}; rows E..S-1 zero
__global__ void __launch_bounds__(256)
router_split_w_kernel(const float* __restrict__ w, __nv_bfloat16* __restrict__ w3, __nv_bfloat16* __restrict__ wbwd, int E, int S,
                      long long d) {
    const long long n = (long long)S * d;
    const __nv_bfloat16 zero = __float2bfloat16_rn(0.f);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / d;
        __nv_bfloat16 hi, mid, lo;
        split3(r < E ? w[i] : 0.f, hi, mid, lo);
        w3[i] = hi; w3[n + i] = mid; w3[2 * n + i] = lo;
        wbwd[i] = hi; wbwd[n + i] = hi; wbwd[2 * n + i] = hi; wbwd[3 * n + i] = mid; wbwd[4 * n + i] = mid; wbwd[5 * n + i] = zero;
    }
}

// ds [T, E] fp32 -> ds6 [T, 6S] = {hi | mid | lo | hi | mid | 0}; also the token-block tables of the split contraction
__global__ void __launch_bounds__(256)
router_split_ds_kernel(const float* __restrict__ ds, __nv_bfloat16* __restrict__ ds6, long long T, int E, int S, int* __restrict__ tables,
                       int splits, long long rows_per_split) {
    if (blockIdx.x == 0 && threadIdx.x <= splits) {
        const int i = threadIdx.x;
        tables[i] = (int)(i * rows_per_split);  // offsets[splits + 1]
        if (i < splits) {
            long long c = T - i * rows_per_split;
            tables[splits + 1 + i] = (int)(c < 0 ? 0 : (c > rows_per_split ? rows_per_split : c));  // counts[splits]
        }
    }
    const long long n = T * S;
    const __nv_bfloat16 zero = __float2bfloat16_rn(0.f);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / S;
        const int e = (int)(i - t * S);
        __nv_bfloat16 hi, mid, lo;
        split3(e < E ? ds[t * E + e] : 0.f, hi, mid, lo);
        __nv_bfloat16* row = ds6 + t * 6 * S;
        row[e] = hi; row[S + e] = mid; row[2 * S + e] = lo; row[3 * S + e] = hi; row[4 * S + e] = mid; row[5 * S + e] = zero;
    }
}

// dW [E, d] = sum over splits and over the three term groups, in a fixed order
__global__ void __launch_bounds__(256)
router_reduce_dw_kernel(const float* __restrict__ partial, float* __restrict__ dw, int E, int S, long long d, int splits) {
    const long long n = (long long)E * d;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long e = i / d, j = i - e * d;
        float acc = 0.f;
        for (int s = 0; s < splits; ++s) {
            const float* slab = partial + (long long)s * 3 * S * d;
            acc += (slab[(2 * S + e) * d + j] + slab[(S + e) * d + j]) + slab[e * d + j];
        }
        dw[i] = acc;
    }
}

// Few tokens (decode): one block per token, a warp per expert in turn, fp32 dot products with the lanes
// striding over the width and a fixed shuffle tree, so the logits are run-to-run identical.  A tile kernel
// would put the whole product on one or two SMs and walk the width serially.
constexpr long long kSmallRouterTokens = 512;
__device__ __forceinline__ float4 load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 load4(const __nv_bfloat16* p) {
    const uint2 v = *reinterpret_cast<const uint2*>(p);
    return make_float4(__uint_as_float(v.x << 16), __uint_as_float(v.x & 0xffff0000u), __uint_as_float(v.y << 16),
                       __uint_as_float(v.y & 0xffff0000u));
}
// grid (tokens, ceil(E / 8)): warp w of block (t, g) computes scores[t, 8 g + w].  Four 16-byte loads of the weight
// row and of the token row are in flight per lane and iteration, so the few round trips to L2 overlap.
template <typename T>
__global__ void __launch_bounds__(256)
router_small_kernel(const T* __restrict__ x, const float* __restrict__ w, float* __restrict__ scores, int E, long long d) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = blockIdx.y * 8 + warp;
    if (e >= E) return;
    const T* row = x + (long long)blockIdx.x * d;
    const float* we = w + (long long)e * d;
    const bool vec = (d & 3) == 0 && (((uintptr_t)row | (uintptr_t)we) & 15u) == 0;
    float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
    if (vec) {
        for (long long j = (long long)lane * 4; j < d; j += 512) {
            float4 wv[4], xv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const long long at = j + 128 * u;
                const bool in = at < d;
                wv[u] = in ? load4(we + at) : make_float4(0.f, 0.f, 0.f, 0.f);
                xv[u] = in ? load4(row + at) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {   // fixed order: the sums do not depend on timing
                a0 = fmaf(xv[u].x, wv[u].x, a0);
                a1 = fmaf(xv[u].y, wv[u].y, a1);
                a2 = fmaf(xv[u].z, wv[u].z, a2);
                a3 = fmaf(xv[u].w, wv[u].w, a3);
            }
        }
    } else {
        for (long long j = lane; j < d; j += 32) a0 = fmaf(Act<T>::load(row + j), we[j], a0);
    }
    float acc = (a0 + a1) + (a2 + a3);
#pragma unroll
    for (int step = 16; step > 0; step >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, step);
    if (lane == 0) scores[(long long)blockIdx.x * E + e] = acc;
}

int elem_grid(long long n) {
    long long blocks = (n + 255) / 256;
    const long long cap = (long long)sm_count() * 8;
    return (int)(blocks > cap ? cap : (blocks < 1 ? 1 : blocks));
}

}  // namespace
}  // namespace qmoe

using namespace qmoe;

extern "C" int64_t qmoe_router_scratch_bytes(int64_t tokens, int32_t experts, int64_t width) {
    const long long simt = simt_router_partials(tokens, experts, width) * 4;
    const long long tc = plan_scratch(tokens, experts, width).total;
    return simt > tc ? simt : tc;
}

extern "C" int64_t qmoe_router_grad_partials(int64_t tokens, int32_t experts, int64_t width) {
    return (qmoe_router_scratch_bytes(tokens, experts, width) + 3) / 4;
}

extern "C" int qmoe_router_forward(uint64_t x, int32_t x_dtype, uint64_t w_router, uint64_t scores, uint64_t scratch,
                                   int64_t tokens, int64_t width, int32_t experts, uint64_t stream_) {
    if (!x || !w_router || !scores) return fail_arg("router_forward: null address");
    if (tokens <= 0 || width <= 0 || experts <= 0) return fail_arg("router_forward: sizes must be positive");
    if (x_dtype != QMOE_F32 && x_dtype != QMOE_BF16) return fail_arg("router_forward: bad dtype %d", x_dtype);
    cudaStream_t stream = (cudaStream_t)stream_;
    if (tokens <= kSmallRouterTokens) {
        TimedScope timed(KC_ROUTER_GEMM, stream);
        if (x_dtype == QMOE_BF16)
            router_small_kernel<__nv_bfloat16><<<dim3((unsigned)tokens, (unsigned)((experts + 7) / 8)), 256, 0, stream>>>((const __nv_bfloat16*)x, (const float*)w_router,
                                                                                   (float*)scores, experts, width);
        else
            router_small_kernel<float><<<dim3((unsigned)tokens, (unsigned)((experts + 7) / 8)), 256, 0, stream>>>((const float*)x, (const float*)w_router,
                                                                             (float*)scores, experts, width);
        QMOE_LAUNCH_CHECK("router_small_kernel");
        return 0;
    }
    if (!tc_router_ok(x_dtype, experts, width, x, scratch))
        return simt_router_logits(x, x_dtype, w_router, scores, tokens, width, experts, stream);
    TimedScope timed(KC_ROUTER_GEMM, stream);
    const RouterScratch r = plan_scratch(tokens, experts, width);
    router_split_w_kernel<<<elem_grid((long long)r.S * width), 256, 0, stream>>>(
        (const float*)w_router, (__nv_bfloat16*)(scratch + r.w3), (__nv_bfloat16*)(scratch + r.wbwd), experts, r.S, width);
    QMOE_LAUNCH_CHECK("router_split_w_kernel");
    return tc_router_forward(x, scratch + r.w3, scores, tokens, width, experts, r.S, stream);
}

extern "C" int qmoe_router_logits(uint64_t x, int32_t x_dtype, uint64_t w_router, uint64_t scores, int64_t tokens,
                                  int64_t width, int32_t experts, uint64_t stream) {
    return qmoe_router_forward(x, x_dtype, w_router, scores, 0, tokens, width, experts, stream);
}

extern "C" int qmoe_router_backward(uint64_t d_scores, uint64_t x, int32_t x_dtype, uint64_t w_router, uint64_t dx_router,
                                    uint64_t d_w_router, uint64_t scratch, int64_t tokens, int64_t width, int32_t experts,
                                    uint64_t stream_) {
    if (!d_scores || !x || !w_router) return fail_arg("router_backward: null address");
    if (tokens <= 0 || width <= 0 || experts <= 0) return fail_arg("router_backward: sizes must be positive");
    if (x_dtype != QMOE_F32 && x_dtype != QMOE_BF16) return fail_arg("router_backward: bad dtype %d", x_dtype);
    cudaStream_t stream = (cudaStream_t)stream_;
    if (!tc_router_ok(x_dtype, experts, width, x, scratch))
        return simt_router_backward(d_scores, x, x_dtype, w_router, dx_router, d_w_router, scratch, tokens, width, experts, stream);
    TimedScope timed(KC_ROUTER_GEMM, stream);
    const RouterScratch r = plan_scratch(tokens, experts, width);
    const int S = r.S;
    int* tables = (int*)(scratch + r.tables);
    // the weight terms are rebuilt here as well: the scratch may have been used by another layer since the forward
    router_split_w_kernel<<<elem_grid((long long)S * width), 256, 0, stream>>>(
        (const float*)w_router, (__nv_bfloat16*)(scratch + r.w3), (__nv_bfloat16*)(scratch + r.wbwd), experts, S, width);
    QMOE_LAUNCH_CHECK("router_split_w_kernel");
    router_split_ds_kernel<<<elem_grid(tokens * S), 256, 0, stream>>>((const float*)d_scores, (__nv_bfloat16*)(scratch + r.ds6),
                                                                      tokens, experts, S, tables, r.splits, r.rows_per_split);
    QMOE_LAUNCH_CHECK("router_split_ds_kernel");
    if (dx_router)
        if (int rc = tc_plain_f32_nn(scratch + r.ds6, scratch + r.wbwd, dx_router, tokens, 6ll * S, width, stream)) return rc;
    if (d_w_router) {
        if (int rc = tc_split_wgrad(scratch + r.ds6, 6ll * S, x, scratch + r.partial, tables, tables + r.splits + 1, r.splits,
                                    tokens, 3ll * S, width, stream)) return rc;
        router_reduce_dw_kernel<<<elem_grid((long long)experts * width), 256, 0, stream>>>(
            (const float*)(scratch + r.partial), (float*)d_w_router, experts, S, width, r.splits);
        QMOE_LAUNCH_CHECK("router_reduce_dw_kernel");
    }
    return 0;
}
