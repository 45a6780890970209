// CUDA-core GEMM (fp32 accumulate) used where the tensor-core path does not apply:
//  * the router (fp32 semantics whatever the activation dtype, skinny N = experts) and its backward;
//  * the expert FFN when activations are fp32 (the 1e-4 parity mode) or the widths are not
//    multiples of 8;
//  * the single-group `qmoe_gemm` of the host-side function table for shapes the tensor-core
//    kernel does not take.
// One generic kernel: arbitrary element strides for both operands, optional second (A2, B2) segment
// accumulated into the same tile, and three ways of grouping by expert.
#include "common.cuh"

namespace qmoe {

namespace {

template <typename T> __device__ __forceinline__ float ldf(const T* p, long long i) { return Act<T>::load(p + i); }

template <typename TA, typename TB, typename TC, int BM, int BN, int TM, int TN>
__global__ void __launch_bounds__(256)
simt_gemm_kernel(SimtGemmArgs g) {
    constexpr int BK = 16;
    static_assert((BM / TM) * (BN / TN) == 256, "256 threads");
    __shared__ float As[BK][BM + 4];
    __shared__ float Bs[BK][BN + 4];
    const int tid = threadIdx.x;
    const long long m0 = (long long)blockIdx.y * BM, n0 = (long long)blockIdx.x * BN;
    long long M = g.M, k_begin = 0, k_end = g.K;
    const TA* A = (const TA*)g.A;
    const TB* B = (const TB*)g.B;
    const TA* A2 = (const TA*)g.A2;
    const TB* B2 = (const TB*)g.B2;
    TC* C = (TC*)g.C;
    if (g.mode == SG_ROWS) {
        M = g.meta[0];
        if (m0 >= M) return;
        const long long e = g.tile_expert[m0 / kRowPad];
        B += e * g.b_slab;
        if (B2) B2 += e * g.b_slab;
    } else if (g.mode == SG_K) {
        const int e = blockIdx.z;
        if (g.counts[e] == 0) return;  // expert received nothing: its slab is left untouched
        k_begin = g.offsets[e];
        k_end = k_begin + g.counts[e];
        C += (long long)e * g.c_slab;
    } else if (g.mode == SG_SPLITK) {
        k_begin = (long long)blockIdx.z * g.k_chunk;
        k_end = k_begin + g.k_chunk < g.K ? k_begin + g.k_chunk : g.K;
        C += (long long)blockIdx.z * g.c_slab;
    }
    if (m0 >= M) return;

    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    const bool a_kfast = g.a_cs == 1, b_kfast = g.b_rs == 1;
    for (int seg = 0; seg < 2; ++seg) {
        const TA* Ap = seg ? A2 : A;
        const TB* Bp = seg ? B2 : B;
        if (!Ap) break;
        for (long long k0 = k_begin; k0 < k_end; k0 += BK) {
#pragma unroll
            for (int l = 0; l < BM * BK / 256; ++l) {
                const int i = tid + l * 256;
                const int kk = a_kfast ? i % BK : i / BM;
                const int mm = a_kfast ? i / BK : i % BM;
                const long long m = m0 + mm, k = k0 + kk;
                As[kk][mm] = (m < M && k < k_end) ? ldf(Ap, m * g.a_rs + k * g.a_cs) : 0.f;
            }
#pragma unroll
            for (int l = 0; l < BN * BK / 256; ++l) {
                const int i = tid + l * 256;
                const int kk = b_kfast ? i % BK : i / BN;
                const int nn = b_kfast ? i / BK : i % BN;
                const long long n = n0 + nn, k = k0 + kk;
                Bs[kk][nn] = (n < g.N && k < k_end) ? ldf(Bp, k * g.b_rs + n * g.b_cs) : 0.f;
            }
            __syncthreads();
#pragma unroll
            for (int kk = 0; kk < BK; ++kk) {
                float a[TM], b[TN];
#pragma unroll
                for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
                for (int j = 0; j < TN; ++j) b[j] = Bs[kk][tx * TN + j];
#pragma unroll
                for (int i = 0; i < TM; ++i)
#pragma unroll
                    for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
            }
            __syncthreads();
        }
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const long long m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const long long n = n0 + tx * TN + j;
            if (n >= g.N) continue;
            TC* dst = C + m * g.ldc + n;
            float v = acc[i][j];
            if (g.accumulate) v += Act<TC>::load(dst);
            Act<TC>::store(dst, v);
        }
    }
}

// sum S partial [S][n] slabs in a fixed order
__global__ void __launch_bounds__(256)
reduce_partials_kernel(const float* __restrict__ partials, float* __restrict__ out, long long n, int splits) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float s = 0.f;
    for (int z = 0; z < splits; ++z) s += partials[(long long)z * n + i];
    out[i] = s;
}

template <typename TA, typename TB, typename TC>
int launch_typed(const SimtGemmArgs& g, long long m_extent, int groups, cudaStream_t stream) {
    if (g.N <= 16) {
        dim3 grid(ceil_div(g.N, 16), ceil_div(m_extent, 128), groups);
        simt_gemm_kernel<TA, TB, TC, 128, 16, 2, 4><<<grid, 256, 0, stream>>>(g);
    } else {
        dim3 grid(ceil_div(g.N, 64), ceil_div(m_extent, 64), groups);
        simt_gemm_kernel<TA, TB, TC, 64, 64, 4, 4><<<grid, 256, 0, stream>>>(g);
    }
    QMOE_LAUNCH_CHECK("simt_gemm_kernel");
    return 0;
}

}  // namespace

// dtype codes: QMOE_F32 / QMOE_BF16 for each of A, B, C.  m_extent = rows the grid must cover.
int launch_simt_gemm(const SimtGemmArgs& g, int a_dtype, int b_dtype, int c_dtype, long long m_extent,
                     int groups, cudaStream_t stream) {
    using bf = __nv_bfloat16;
    const int key = (a_dtype << 2) | (b_dtype << 1) | c_dtype;
    switch (key) {
        case 0: return launch_typed<float, float, float>(g, m_extent, groups, stream);
        case 1: return launch_typed<float, float, bf>(g, m_extent, groups, stream);
        case 2: return launch_typed<float, bf, float>(g, m_extent, groups, stream);
        case 3: return launch_typed<float, bf, bf>(g, m_extent, groups, stream);
        case 4: return launch_typed<bf, float, float>(g, m_extent, groups, stream);
        case 5: return launch_typed<bf, float, bf>(g, m_extent, groups, stream);
        case 6: return launch_typed<bf, bf, float>(g, m_extent, groups, stream);
        case 7: return launch_typed<bf, bf, bf>(g, m_extent, groups, stream);
    }
    return fail_arg("bad dtype combination");
}

int launch_reduce_partials(const float* partials, float* out, long long n, int splits, cudaStream_t stream) {
    reduce_partials_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(partials, out, n, splits);
    QMOE_LAUNCH_CHECK("reduce_partials_kernel");
    return 0;
}

}  // namespace qmoe

namespace qmoe {
namespace {
constexpr long long kRouterSplitTokens = 2048;
}

int simt_router_logits(uint64_t x, int32_t x_dtype, uint64_t w_router, uint64_t scores, int64_t tokens, int64_t width,
                       int32_t experts, cudaStream_t stream) {
    TimedScope timed(KC_ROUTER_GEMM, stream);
    SimtGemmArgs g = {};
    g.A = (const void*)x; g.B = (const void*)w_router; g.C = (void*)scores;
    g.M = tokens; g.N = experts; g.K = width;
    g.a_rs = width; g.a_cs = 1;
    g.b_rs = 1; g.b_cs = width;  // B(k, n) = W[n, k]
    g.ldc = experts;
    g.mode = SG_PLAIN;
    return launch_simt_gemm(g, x_dtype, QMOE_F32, QMOE_F32, tokens, 1, stream);
}

long long simt_router_partials(int64_t tokens, int32_t experts, int64_t width) {
    const int64_t splits = (tokens + kRouterSplitTokens - 1) / kRouterSplitTokens;
    return splits * experts * width;
}

int simt_router_backward(uint64_t d_scores, uint64_t x, int32_t x_dtype, uint64_t w_router, uint64_t dx_router,
                         uint64_t d_w_router, uint64_t partials, int64_t tokens, int64_t width, int32_t experts,
                         cudaStream_t stream) {
    TimedScope timed(KC_ROUTER_GEMM, stream);
    if (dx_router) {  // [T, d] = d_scores[T, E] . W[E, d]
        SimtGemmArgs g = {};
        g.A = (const void*)d_scores; g.B = (const void*)w_router; g.C = (void*)dx_router;
        g.M = tokens; g.N = width; g.K = experts;
        g.a_rs = experts; g.a_cs = 1;
        g.b_rs = width; g.b_cs = 1;
        g.ldc = width;
        g.mode = SG_PLAIN;
        if (int rc = launch_simt_gemm(g, QMOE_F32, QMOE_F32, QMOE_F32, tokens, 1, stream)) return rc;
    }
    if (d_w_router) {  // [E, d] = d_scores^T[E, T] . x[T, d], split over tokens, reduced in fixed order
        if (!partials) return fail_arg("router_backward: scratch is null");
        const int splits = (int)((tokens + kRouterSplitTokens - 1) / kRouterSplitTokens);
        SimtGemmArgs g = {};
        g.A = (const void*)d_scores; g.B = (const void*)x; g.C = (void*)partials;
        g.M = experts; g.N = width; g.K = tokens;
        g.a_rs = 1; g.a_cs = experts;  // A(m = e, k = t) = d_scores[t, e]
        g.b_rs = width; g.b_cs = 1;
        g.ldc = width;
        g.mode = SG_SPLITK;
        g.k_chunk = kRouterSplitTokens;
        g.c_slab = (long long)experts * width;
        if (int rc = launch_simt_gemm(g, QMOE_F32, x_dtype, QMOE_F32, experts, splits, stream)) return rc;
        if (int rc = launch_reduce_partials((const float*)partials, (float*)d_w_router,
                                            (long long)experts * width, splits, stream)) return rc;
    }
    return 0;
}

}  // namespace qmoe
