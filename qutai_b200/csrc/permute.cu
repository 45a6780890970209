// Memory-bound stages of the MoE layer: permute (dispatch gather), weighted combine, their
// backwards, SwiGLU element-wise forward/backward, fp32->bf16 weight cast, SiLU.
//
// One warp moves one row; each lane moves 16-byte vectors (8 bf16 or 4 fp32) and keeps several
// independent loads in flight before the first store.  When the row pitch is not a multiple of
// 16 bytes (or a base address is not 16-byte aligned) the scalar instantiation is used instead.
#include <initializer_list>

#include "common.cuh"

namespace qmoe {

namespace {

constexpr int kThreads = 256;
constexpr int kWarpsPerBlock = kThreads / 32;

__device__ __forceinline__ void st16(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }
// streaming variants: data that is read or written once should not displace reusable lines in L2
__device__ __forceinline__ uint4 ld16_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

// ---- permute: dispatched[dest_row[t, s]] = x[t] for every slot, pads zero ------------------------
// Organised by TOKEN: a warp reads one token row once and writes its k copies, so the source is
// read T*d instead of A*d times (the k copies of a token lie far apart in the dispatched layout and
// would miss L2).  Pad rows are zeroed afterwards by the warps that find row_source[r] < 0.
template <typename T, bool VEC, int KMAX>
__global__ void __launch_bounds__(kThreads)
permute_kernel(const T* __restrict__ x, T* __restrict__ out, const int* __restrict__ dest_row,
               const int* __restrict__ row_source, const int* __restrict__ meta, long long tokens, int k,
               long long width) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * kWarpsPerBlock;
    for (long long t = warp; t < tokens; t += nwarps) {
        long long rows[KMAX];
#pragma unroll
        for (int s = 0; s < KMAX; ++s) rows[s] = s < k ? dest_row[t * k + s] : 0;
        const T* src = x + t * width;
        if constexpr (VEC) {
            constexpr int N = Vec16<T>::N;
            const int chunks = (int)(width / N);
            int c = lane;
            for (; c + 32 < chunks; c += 64) {
                const uint4 v0 = ld16_stream(src + (long long)c * N), v1 = ld16_stream(src + (long long)(c + 32) * N);
#pragma unroll
                for (int s = 0; s < KMAX; ++s)
                    if (s < k) {
                        st16(out + rows[s] * width + (long long)c * N, v0);
                        st16(out + rows[s] * width + (long long)(c + 32) * N, v1);
                    }
            }
            for (; c < chunks; c += 32) {
                const uint4 v0 = ld16_stream(src + (long long)c * N);
#pragma unroll
                for (int s = 0; s < KMAX; ++s)
                    if (s < k) st16(out + rows[s] * width + (long long)c * N, v0);
            }
        } else {
            for (long long c = lane; c < width; c += 32) {
                const T v = src[c];
                for (int s = 0; s < k; ++s) out[rows[s] * width + c] = v;
            }
        }
    }
    const int rows_used = meta[0];
    for (long long r = warp; r < rows_used; r += nwarps) {
        if (row_source[r] >= 0) continue;
        T* dst = out + r * width;
        if constexpr (VEC) {
            constexpr int N = Vec16<T>::N;
            for (int c = lane; c < (int)(width / N); c += 32) st16(dst + (long long)c * N, make_uint4(0, 0, 0, 0));
        } else {
            for (long long c = lane; c < width; c += 32) Act<T>::store(dst + c, 0.f);
        }
    }
}

// ---- combine: out[t] = sum_s w[t,s] * y[dest_row[t,s]] ----------------------------------------
template <typename T, bool VEC, int KMAX>
__global__ void __launch_bounds__(kThreads)
combine_kernel(const T* __restrict__ y, const float* __restrict__ gate_w, const int* __restrict__ dest_row,
               T* __restrict__ out, long long tokens, int k, long long width) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * kWarpsPerBlock;
    for (long long t = warp; t < tokens; t += nwarps) {
        int rows[KMAX];
        float w[KMAX];
#pragma unroll
        for (int s = 0; s < KMAX; ++s) {
            rows[s] = s < k ? dest_row[t * k + s] : 0;
            w[s] = s < k ? gate_w[t * k + s] : 0.f;
        }
        T* dst = out + t * width;
        if constexpr (VEC) {
            constexpr int N = Vec16<T>::N;
            const int chunks = (int)(width / N);
            for (int c = lane; c < chunks; c += 32) {
                uint4 v[KMAX];
#pragma unroll
                for (int s = 0; s < KMAX; ++s)
                    if (s < k) v[s] = ld16_stream(y + (long long)rows[s] * width + (long long)c * N);
                float acc[N];
#pragma unroll
                for (int i = 0; i < N; ++i) acc[i] = 0.f;
#pragma unroll
                for (int s = 0; s < KMAX; ++s)
                    if (s < k) {
                        float f[N];
                        Vec16<T>::unpack(v[s], f);
#pragma unroll
                        for (int i = 0; i < N; ++i) acc[i] = fmaf(w[s], f[i], acc[i]);
                    }
                st16(dst + (long long)c * N, Vec16<T>::pack(acc));
            }
        } else {
            for (long long c = lane; c < width; c += 32) {
                float acc = 0.f;
                for (int s = 0; s < k; ++s) acc = fmaf(w[s], Act<T>::load(y + (long long)rows[s] * width + c), acc);
                Act<T>::store(dst + c, acc);
            }
        }
    }
}

// ---- combine backward: dy[dest_row[t, s]] = g[t] * w[t, s];  dw[t, s] = <g[t], y[dest_row[t, s]]> ----
// Organised by TOKEN like the permute: g[t] is read once for its k slots.
template <typename T, bool VEC, int KMAX>
__global__ void __launch_bounds__(kThreads)
combine_backward_kernel(const T* __restrict__ g, const T* __restrict__ y, const float* __restrict__ gate_w,
                        const int* __restrict__ dest_row, const int* __restrict__ row_source,
                        const int* __restrict__ meta, T* __restrict__ dy, float* __restrict__ dw, long long tokens,
                        int k, long long width) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * kWarpsPerBlock;
    for (long long t = warp; t < tokens; t += nwarps) {
        long long rows[KMAX];
        float w[KMAX], dot[KMAX];
#pragma unroll
        for (int s = 0; s < KMAX; ++s) {
            rows[s] = s < k ? dest_row[t * k + s] : 0;
            w[s] = s < k ? gate_w[t * k + s] : 0.f;
            dot[s] = 0.f;
        }
        const T* gs = g + t * width;
        if constexpr (VEC) {
            constexpr int N = Vec16<T>::N;
            const int chunks = (int)(width / N);
            for (int c = lane; c < chunks; c += 32) {
                float fg[N];
                Vec16<T>::unpack(ld16_stream(gs + (long long)c * N), fg);
                uint4 v[KMAX];
#pragma unroll
                for (int s = 0; s < KMAX; ++s)
                    if (s < k) v[s] = ld16_stream(y + rows[s] * width + (long long)c * N);
#pragma unroll
                for (int s = 0; s < KMAX; ++s)
                    if (s < k) {
                        float fy[N], o[N];
                        Vec16<T>::unpack(v[s], fy);
#pragma unroll
                        for (int i = 0; i < N; ++i) { dot[s] = fmaf(fg[i], fy[i], dot[s]); o[i] = fg[i] * w[s]; }
                        st16(dy + rows[s] * width + (long long)c * N, Vec16<T>::pack(o));
                    }
            }
        } else {
            for (long long c = lane; c < width; c += 32) {
                const float gv = Act<T>::load(gs + c);
                for (int s = 0; s < k; ++s) {
                    dot[s] = fmaf(gv, Act<T>::load(y + rows[s] * width + c), dot[s]);
                    Act<T>::store(dy + rows[s] * width + c, gv * w[s]);
                }
            }
        }
#pragma unroll
        for (int s = 0; s < KMAX; ++s)
            if (s < k) {
                const float total = warp_sum(dot[s]);
                if (lane == 0) dw[t * k + s] = total;
            }
    }
    const int rows_used = meta[0];
    for (long long r = warp; r < rows_used; r += nwarps) {
        if (row_source[r] >= 0) continue;
        T* dst = dy + r * width;
        if constexpr (VEC) {
            constexpr int N = Vec16<T>::N;
            for (int c = lane; c < (int)(width / N); c += 32) st16(dst + (long long)c * N, make_uint4(0, 0, 0, 0));
        } else {
            for (long long c = lane; c < width; c += 32) Act<T>::store(dst + c, 0.f);
        }
    }
}

// ---- unpermute-reduce: dx[t] = sum_s d_dispatched[dest_row[t,s]] (+ extra[t]) -----------------
template <typename T, bool VEC, int KMAX>
__global__ void __launch_bounds__(kThreads)
unpermute_kernel(const T* __restrict__ dxd, const float* __restrict__ extra, const int* __restrict__ dest_row,
                 T* __restrict__ dx, long long tokens, int k, long long width) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * kWarpsPerBlock;
    for (long long t = warp; t < tokens; t += nwarps) {
        int rows[KMAX];
#pragma unroll
        for (int s = 0; s < KMAX; ++s) rows[s] = s < k ? dest_row[t * k + s] : 0;
        T* dst = dx + t * width;
        if constexpr (VEC) {
            constexpr int N = Vec16<T>::N;
            const int chunks = (int)(width / N);
            for (int c = lane; c < chunks; c += 32) {
                uint4 v[KMAX];
#pragma unroll
                for (int s = 0; s < KMAX; ++s)
                    if (s < k) v[s] = ld16_stream(dxd + (long long)rows[s] * width + (long long)c * N);
                float acc[N];
                if (extra) {
                    const float* ex = extra + t * width + (long long)c * N;
#pragma unroll
                    for (int i = 0; i < N; i += 4) {
                        const float4 e4 = *reinterpret_cast<const float4*>(ex + i);
                        acc[i] = e4.x; acc[i + 1] = e4.y; acc[i + 2] = e4.z; acc[i + 3] = e4.w;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < N; ++i) acc[i] = 0.f;
                }
#pragma unroll
                for (int s = 0; s < KMAX; ++s)
                    if (s < k) {
                        float f[N];
                        Vec16<T>::unpack(v[s], f);
#pragma unroll
                        for (int i = 0; i < N; ++i) acc[i] += f[i];
                    }
                st16(dst + (long long)c * N, Vec16<T>::pack(acc));
            }
        } else {
            for (long long c = lane; c < width; c += 32) {
                float acc = extra ? extra[t * width + c] : 0.f;
                for (int s = 0; s < k; ++s) acc += Act<T>::load(dxd + (long long)rows[s] * width + c);
                Act<T>::store(dst + c, acc);
            }
        }
    }
}

// ---- SwiGLU element-wise over the dispatched rows (used by the CUDA-core GEMM path) -----------
// Rounding points follow the upstream activations: silu(G) is stored in the activation dtype
// before the multiply (src/qutai/lm/layers.py:311 builds it from two separate kernels).
template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_kernel(const T* __restrict__ G, const T* __restrict__ U, T* __restrict__ H,
              const int* __restrict__ meta, long long hidden) {
    const long long n = (long long)meta[0] * hidden;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float g = Act<T>::load(G + i), u = Act<T>::load(U + i);
        T act;
        Act<T>::store(&act, g * sigmoid_stable(g));
        Act<T>::store(H + i, Act<T>::load(&act) * u);
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
swiglu_backward_kernel(const T* __restrict__ dH, const T* __restrict__ G, const T* __restrict__ U,
                       T* __restrict__ dG, T* __restrict__ dU, const int* __restrict__ meta, long long hidden) {
    const long long n = (long long)meta[0] * hidden;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float dh = Act<T>::load(dH + i), g = Act<T>::load(G + i), u = Act<T>::load(U + i);
        const float s = sigmoid_stable(g);
        T act, ds;
        Act<T>::store(&act, g * s);
        Act<T>::store(dU + i, dh * Act<T>::load(&act));
        Act<T>::store(&ds, dh * u);
        Act<T>::store(dG + i, Act<T>::load(&ds) * s * (1.f + g * (1.f - s)));
    }
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
silu_kernel(const T* __restrict__ v, const T* __restrict__ g, T* __restrict__ out, long long n, int backward) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const float x = Act<T>::load(v + i);
        const float s = sigmoid_stable(x);
        Act<T>::store(out + i, backward ? Act<T>::load(g + i) * s * (1.f + x * (1.f - s)) : x * s);
    }
}

__global__ void __launch_bounds__(kThreads)
cast_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst, long long n) {
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long n8 = n / 8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += stride) {
        const uint4 a = ld16_stream(src + i * 8), b = ld16_stream(src + i * 8 + 4);
        float f[8];
        Vec16<float>::unpack(a, f);
        Vec16<float>::unpack(b, f + 4);
        st16(dst + i * 8, Vec16<__nv_bfloat16>::pack(f));
    }
    for (long long i = n8 * 8 + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        dst[i] = __float2bfloat16_rn(src[i]);
}

template <typename T>
__global__ void __launch_bounds__(kThreads)
add_kernel(const T* __restrict__ a, const T* __restrict__ b, T* __restrict__ out, long long n) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        Act<T>::store(out + i, Act<T>::load(a + i) + Act<T>::load(b + i));
}

// counter-based generator: a 64-bit mix of (seed, index) gives two uniforms, Box-Muller one normal
__device__ __forceinline__ unsigned long long mix64(unsigned long long z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}
template <typename T>
__global__ void __launch_bounds__(kThreads)
normal_fill_kernel(T* __restrict__ out, long long n, float mean, float std, unsigned long long seed) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const unsigned long long h = mix64(mix64(seed) ^ (unsigned long long)i);
        const float u1 = ((float)(h >> 40) + 1.0f) * (1.0f / 16777216.0f);       // (0, 1]
        const float u2 = (float)((h >> 16) & 0xFFFFFFull) * (1.0f / 16777216.0f); // [0, 1)
        const float z = sqrtf(-2.0f * logf(u1)) * cospif(2.0f * u2);
        Act<T>::store(out + i, mean + std * z);
    }
}

bool aligned16(uint64_t p) { return (p & 15u) == 0; }

template <typename T>
bool can_vec(long long width, std::initializer_list<uint64_t> ptrs) {
    if ((width * (long long)sizeof(T)) % 16) return false;
    for (uint64_t p : ptrs)
        if (!aligned16(p)) return false;
    return true;
}

int grid_for_rows(long long rows) {
    long long blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const long long cap = (long long)sm_count() * 8;  // 8 resident 256-thread blocks per SM
    if (blocks > cap) blocks = cap;
    return (int)(blocks < 1 ? 1 : blocks);
}

int grid_for_elems(long long n) {
    long long blocks = (n + kThreads - 1) / kThreads;
    const long long cap = (long long)sm_count() * 8;
    if (blocks > cap) blocks = cap;
    return (int)(blocks < 1 ? 1 : blocks);
}

int check_dtype(int dtype) {
    if (dtype != QMOE_F32 && dtype != QMOE_BF16) return fail_arg("dtype must be QMOE_F32 or QMOE_BF16 (got %d)", dtype);
    return 0;
}

}  // namespace

// internal entry points shared with the layer driver ------------------------------------------
int launch_swiglu(const qmoe_route_t* r, uint64_t g, uint64_t u, uint64_t h, int dtype, long long hidden,
                  cudaStream_t stream) {
    TimedScope timed(KC_SWIGLU, stream);
    const int grid = grid_for_elems(r->rows_bound * hidden);
    if (dtype == QMOE_BF16)
        swiglu_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>((const __nv_bfloat16*)g, (const __nv_bfloat16*)u,
                                                                     (__nv_bfloat16*)h, (const int*)r->meta, hidden);
    else
        swiglu_kernel<float><<<grid, kThreads, 0, stream>>>((const float*)g, (const float*)u, (float*)h,
                                                             (const int*)r->meta, hidden);
    QMOE_LAUNCH_CHECK("swiglu_kernel");
    return 0;
}

int launch_swiglu_backward(const qmoe_route_t* r, uint64_t dh, uint64_t g, uint64_t u, uint64_t dg, uint64_t du,
                           int dtype, long long hidden, cudaStream_t stream) {
    TimedScope timed(KC_SWIGLU, stream);
    const int grid = grid_for_elems(r->rows_bound * hidden);
    if (dtype == QMOE_BF16)
        swiglu_backward_kernel<__nv_bfloat16><<<grid, kThreads, 0, stream>>>(
            (const __nv_bfloat16*)dh, (const __nv_bfloat16*)g, (const __nv_bfloat16*)u, (__nv_bfloat16*)dg,
            (__nv_bfloat16*)du, (const int*)r->meta, hidden);
    else
        swiglu_backward_kernel<float><<<grid, kThreads, 0, stream>>>((const float*)dh, (const float*)g, (const float*)u,
                                                                      (float*)dg, (float*)du, (const int*)r->meta, hidden);
    QMOE_LAUNCH_CHECK("swiglu_backward_kernel");
    return 0;
}

}  // namespace qmoe

using namespace qmoe;

extern "C" int qmoe_permute(const qmoe_route_t* r, uint64_t x, uint64_t out, int32_t dtype, int64_t width,
                            uint64_t stream_) {
    if (int rc = route_check(r)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (!x || !out || width <= 0) return fail_arg("permute: null address or non-positive width");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_PERMUTE, stream);
    const bool vec = dtype == QMOE_BF16 ? can_vec<__nv_bfloat16>(width, {x, out}) : can_vec<float>(width, {x, out});
    // enough warps for the tokens and for zeroing up to experts * 127 pad rows
    const int grid = grid_for_rows(r->tokens > (long long)r->experts * 64 ? r->tokens : (long long)r->experts * 64);
#define ARGS(T) <<<grid, kThreads, 0, stream>>>((const T*)x, (T*)out, (const int*)r->dest_row, (const int*)r->row_source, (const int*)r->meta, (long long)r->tokens, r->top_k, (long long)width)
#define BY_K(T, V)                                                  \
    do {                                                            \
        if (r->top_k <= 1) permute_kernel<T, V, 1> ARGS(T);         \
        else if (r->top_k <= 2) permute_kernel<T, V, 2> ARGS(T);    \
        else if (r->top_k <= 4) permute_kernel<T, V, 4> ARGS(T);    \
        else if (r->top_k <= 6) permute_kernel<T, V, 6> ARGS(T);    \
        else permute_kernel<T, V, 8> ARGS(T);                       \
    } while (0)
    if (dtype == QMOE_BF16) { if (vec) BY_K(__nv_bfloat16, true); else BY_K(__nv_bfloat16, false); }
    else { if (vec) BY_K(float, true); else BY_K(float, false); }
#undef BY_K
#undef ARGS
    QMOE_LAUNCH_CHECK("permute_kernel");
    return 0;
}

extern "C" int qmoe_combine(const qmoe_route_t* r, uint64_t y, uint64_t out, int32_t dtype, int64_t width,
                            uint64_t stream_) {
    if (int rc = route_check(r)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (!y || !out || width <= 0) return fail_arg("combine: null address or non-positive width");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_COMBINE, stream);
    const bool vec = dtype == QMOE_BF16 ? can_vec<__nv_bfloat16>(width, {y, out}) : can_vec<float>(width, {y, out});
    const int grid = grid_for_rows(r->tokens);
#define ARGS(T) <<<grid, kThreads, 0, stream>>>((const T*)y, (const float*)r->gate_weights, (const int*)r->dest_row, (T*)out, (long long)r->tokens, r->top_k, (long long)width)
#define BY_K(T, V)                                                  \
    do {                                                            \
        if (r->top_k <= 1) combine_kernel<T, V, 1> ARGS(T);         \
        else if (r->top_k <= 2) combine_kernel<T, V, 2> ARGS(T);    \
        else if (r->top_k <= 4) combine_kernel<T, V, 4> ARGS(T);    \
        else if (r->top_k <= 6) combine_kernel<T, V, 6> ARGS(T);    \
        else combine_kernel<T, V, 8> ARGS(T);                       \
    } while (0)
    if (dtype == QMOE_BF16) { if (vec) BY_K(__nv_bfloat16, true); else BY_K(__nv_bfloat16, false); }
    else { if (vec) BY_K(float, true); else BY_K(float, false); }
#undef BY_K
#undef ARGS
    QMOE_LAUNCH_CHECK("combine_kernel");
    return 0;
}

extern "C" int qmoe_combine_backward(const qmoe_route_t* r, uint64_t g, uint64_t y, uint64_t dy, uint64_t dw,
                                     int32_t dtype, int64_t width, uint64_t stream_) {
    if (int rc = route_check(r)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (!g || !y || !dy || !dw || width <= 0) return fail_arg("combine_backward: null address or non-positive width");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_COMBINE_BWD, stream);
    const bool vec = dtype == QMOE_BF16 ? can_vec<__nv_bfloat16>(width, {g, y, dy}) : can_vec<float>(width, {g, y, dy});
    const int grid = grid_for_rows(r->tokens > (long long)r->experts * 64 ? r->tokens : (long long)r->experts * 64);
#define ARGS(T) <<<grid, kThreads, 0, stream>>>((const T*)g, (const T*)y, (const float*)r->gate_weights, (const int*)r->dest_row, (const int*)r->row_source, (const int*)r->meta, (T*)dy, (float*)dw, (long long)r->tokens, r->top_k, (long long)width)
#define BY_K(T, V)                                                           \
    do {                                                                     \
        if (r->top_k <= 1) combine_backward_kernel<T, V, 1> ARGS(T);         \
        else if (r->top_k <= 2) combine_backward_kernel<T, V, 2> ARGS(T);    \
        else if (r->top_k <= 4) combine_backward_kernel<T, V, 4> ARGS(T);    \
        else if (r->top_k <= 6) combine_backward_kernel<T, V, 6> ARGS(T);    \
        else combine_backward_kernel<T, V, 8> ARGS(T);                       \
    } while (0)
    if (dtype == QMOE_BF16) { if (vec) BY_K(__nv_bfloat16, true); else BY_K(__nv_bfloat16, false); }
    else { if (vec) BY_K(float, true); else BY_K(float, false); }
#undef BY_K
#undef ARGS
    QMOE_LAUNCH_CHECK("combine_backward_kernel");
    return 0;
}

extern "C" int qmoe_unpermute_reduce(const qmoe_route_t* r, uint64_t dxd, uint64_t extra, uint64_t dx,
                                     int32_t dtype, int64_t width, uint64_t stream_) {
    if (int rc = route_check(r)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (!dxd || !dx || width <= 0) return fail_arg("unpermute_reduce: null address or non-positive width");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_UNPERMUTE, stream);
    bool vec = dtype == QMOE_BF16 ? can_vec<__nv_bfloat16>(width, {dxd, dx}) : can_vec<float>(width, {dxd, dx});
    if (extra && (!aligned16(extra) || (width * 4) % 16)) vec = false;
    const int grid = grid_for_rows(r->tokens);
#define ARGS(T) <<<grid, kThreads, 0, stream>>>((const T*)dxd, (const float*)extra, (const int*)r->dest_row, (T*)dx, (long long)r->tokens, r->top_k, (long long)width)
#define BY_K(T, V)                                                    \
    do {                                                              \
        if (r->top_k <= 1) unpermute_kernel<T, V, 1> ARGS(T);         \
        else if (r->top_k <= 2) unpermute_kernel<T, V, 2> ARGS(T);    \
        else if (r->top_k <= 4) unpermute_kernel<T, V, 4> ARGS(T);    \
        else if (r->top_k <= 6) unpermute_kernel<T, V, 6> ARGS(T);    \
        else unpermute_kernel<T, V, 8> ARGS(T);                       \
    } while (0)
    if (dtype == QMOE_BF16) { if (vec) BY_K(__nv_bfloat16, true); else BY_K(__nv_bfloat16, false); }
    else { if (vec) BY_K(float, true); else BY_K(float, false); }
#undef BY_K
#undef ARGS
    QMOE_LAUNCH_CHECK("unpermute_kernel");
    return 0;
}

extern "C" int qmoe_cast_bf16(uint64_t src, uint64_t dst, int64_t n, uint64_t stream_) {
    if (!src || !dst || n < 0) return fail_arg("cast_bf16: null address or negative size");
    if (!aligned16(src) || !aligned16(dst)) return fail_arg("cast_bf16: addresses must be 16-byte aligned");
    if (n == 0) return 0;
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_CAST, stream);
    cast_bf16_kernel<<<grid_for_elems(n / 8 + 1), kThreads, 0, stream>>>((const float*)src, (__nv_bfloat16*)dst, n);
    QMOE_LAUNCH_CHECK("cast_bf16_kernel");
    return 0;
}

extern "C" int qmoe_silu(uint64_t values, uint64_t gradient, uint64_t out, int32_t dtype, int64_t n,
                         int32_t backward, uint64_t stream_) {
    if (int rc = check_dtype(dtype)) return rc;
    if (!values || !out || n < 0 || (backward && !gradient)) return fail_arg("silu: null address or negative size");
    if (n == 0) return 0;
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_SWIGLU, stream);
    if (dtype == QMOE_BF16)
        silu_kernel<__nv_bfloat16><<<grid_for_elems(n), kThreads, 0, stream>>>(
            (const __nv_bfloat16*)values, (const __nv_bfloat16*)gradient, (__nv_bfloat16*)out, n, backward);
    else
        silu_kernel<float><<<grid_for_elems(n), kThreads, 0, stream>>>((const float*)values, (const float*)gradient,
                                                                        (float*)out, n, backward);
    QMOE_LAUNCH_CHECK("silu_kernel");
    return 0;
}

extern "C" int qmoe_add(uint64_t a, uint64_t b, uint64_t out, int32_t dtype, int64_t n, uint64_t stream_) {
    if (int rc = check_dtype(dtype)) return rc;
    if (!a || !b || !out || n < 0) return fail_arg("add: null address or negative size");
    if (n == 0) return 0;
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_ELEMENTWISE, stream);
    if (dtype == QMOE_BF16)
        add_kernel<__nv_bfloat16><<<grid_for_elems(n), kThreads, 0, stream>>>((const __nv_bfloat16*)a, (const __nv_bfloat16*)b,
                                                                               (__nv_bfloat16*)out, n);
    else
        add_kernel<float><<<grid_for_elems(n), kThreads, 0, stream>>>((const float*)a, (const float*)b, (float*)out, n);
    QMOE_LAUNCH_CHECK("add_kernel");
    return 0;
}

extern "C" int qmoe_normal_fill(uint64_t out, int32_t dtype, int64_t n, double mean, double std, uint64_t seed,
                                uint64_t stream_) {
    if (int rc = check_dtype(dtype)) return rc;
    if (!out || n < 0) return fail_arg("normal_fill: null address or negative size");
    if (n == 0) return 0;
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_OTHER, stream);
    if (dtype == QMOE_BF16)
        normal_fill_kernel<__nv_bfloat16><<<grid_for_elems(n), kThreads, 0, stream>>>((__nv_bfloat16*)out, n, (float)mean,
                                                                                       (float)std, seed);
    else
        normal_fill_kernel<float><<<grid_for_elems(n), kThreads, 0, stream>>>((float*)out, n, (float)mean, (float)std, seed);
    QMOE_LAUNCH_CHECK("normal_fill_kernel");
    return 0;
}

// ---- row gather: dst[i, :] = src[index[i], :] (16-byte pieces; expert-indexed tables of a few hundred KB) ----
namespace qmoe {
namespace {
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, const int* __restrict__ index, int rows,
                   long long row_vecs, int src_rows) {
    const long long total = (long long)rows * row_vecs;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int row = (int)(i / row_vecs);
        const int from = index[row];
        if (from < 0 || from >= src_rows) continue;  // a bad table never becomes a bad address
        dst[i] = src[(long long)from * row_vecs + (i - (long long)row * row_vecs)];
    }
}
__global__ void __launch_bounds__(256)
gather_words_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst, const int* __restrict__ index, int rows,
                    long long row_words, int src_rows) {
    const long long total = (long long)rows * row_words;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int row = (int)(i / row_words);
        const int from = index[row];
        if (from < 0 || from >= src_rows) continue;
        dst[i] = src[(long long)from * row_words + (i - (long long)row * row_words)];
    }
}
}  // namespace
}  // namespace qmoe

extern "C" int qmoe_gather_rows(uint64_t src, uint64_t dst, uint64_t index, int32_t rows, int32_t src_rows, int64_t row_bytes,
                                uint64_t stream_) {
    if (!src || !dst || !index) return fail_arg("gather_rows: null address");
    if (src == dst) return fail_arg("gather_rows: the output must not alias the input");
    if (rows <= 0 || src_rows <= 0 || row_bytes <= 0 || row_bytes % 4) return fail_arg("gather_rows: rows must be positive and a multiple of 4 bytes");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_OTHER, stream);
    if (row_bytes % 16 == 0 && !((src | dst) & 15u)) {
        const long long total = (long long)rows * (row_bytes / 16);
        gather_rows_kernel<<<(int)((total + 255) / 256 > 1184 ? 1184 : (total + 255) / 256), 256, 0, stream>>>(
            (const uint4*)src, (uint4*)dst, (const int*)index, rows, row_bytes / 16, src_rows);
    } else {
        const long long total = (long long)rows * (row_bytes / 4);
        gather_words_kernel<<<(int)((total + 255) / 256 > 1184 ? 1184 : (total + 255) / 256), 256, 0, stream>>>(
            (const uint32_t*)src, (uint32_t*)dst, (const int*)index, rows, row_bytes / 4, src_rows);
    }
    QMOE_LAUNCH_CHECK("gather_rows_kernel");
    return 0;
}
