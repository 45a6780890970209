// The small memory-bound operations around attention and the feed-forward half of a decoder block, with upstream's
// meaning of every argument (src/qutai/backends/cuda_lm.py, kernels src/qutai/backends/cuda/lm.cu:11-64, CPU statements
// src/qutai/backends/cpu_lm.py:54-140): RMS norm and its backward, rotary position embedding, the token embedding and
// its backward.  Upstream launches one 256-thread block per row (norm) or one thread per element with scalar accesses;
// here a warp owns a row and moves 16 or 32 bytes per lane per access in the norm, the norm weight's gradient is reduced in a fixed
// order (no floating-point atomics), and the embedding's backward walks each token's positions in order, as
// upstream's does, so every result is the same on every run.
#include "common.cuh"

namespace qmoe {
namespace {

constexpr int kThreads = 256;
constexpr int kWarpsPerBlock = kThreads / 32;
constexpr int kSlabRows = 64;          // rows of one block of the norm weight's gradient

int row_grid(long long rows) {
    const long long blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    return (int)(blocks > 8ll * 148 ? 8 * 148 : (blocks < 1 ? 1 : blocks));
}
int flat_grid(long long n) {
    const long long blocks = (n + kThreads - 1) / kThreads;
    return (int)(blocks > 8ll * 148 ? 8 * 148 : (blocks < 1 ? 1 : blocks));
}

// eight consecutive elements per lane and access: 16 bytes of bf16, 32 bytes of fp32
__device__ __forceinline__ void load8(const float* p, float* f) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* f) { Vec16<__nv_bfloat16>::unpack(*reinterpret_cast<const uint4*>(p), f); }
__device__ __forceinline__ void store8(float* p, const float* f) {
    *reinterpret_cast<float4*>(p) = make_float4(f[0], f[1], f[2], f[3]);
    *reinterpret_cast<float4*>(p + 4) = make_float4(f[4], f[5], f[6], f[7]);
}
__device__ __forceinline__ void store8(__nv_bfloat16* p, const float* f) { *reinterpret_cast<uint4*>(p) = Vec16<__nv_bfloat16>::pack(f); }

// out[r, :] = x[r, :] * inverse[r] * weight, inverse[r] = 1 / sqrt(mean(x[r, :]^2) + eps).  VEC: width a multiple of 8 and
// 32-byte aligned rows.
template <typename TX, typename TO, bool VEC>
__global__ void __launch_bounds__(kThreads)
rms_norm_kernel(const TX* __restrict__ x, const float* __restrict__ weight, TO* __restrict__ out, float* __restrict__ inverse,
                long long rows, long long width, float eps) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * kWarpsPerBlock;
    for (long long r = warp; r < rows; r += nwarps) {
        const TX* src = x + r * width;
        TO* dst = out + r * width;
        float total = 0.f;
        if (VEC) {
            for (long long c = lane * 8; c < width; c += 256) {
                float f[8];
                load8(src + c, f);
#pragma unroll
                for (int e = 0; e < 8; ++e) total = fmaf(f[e], f[e], total);
            }
        } else {
            for (long long c = lane; c < width; c += 32) {
                const float v = Act<TX>::load(src + c);
                total = fmaf(v, v, total);
            }
        }
        total = warp_sum(total);
        const float inv = rsqrtf(total / (float)width + eps);
        if (lane == 0) inverse[r] = inv;
        if (VEC) {
            for (long long c = lane * 8; c < width; c += 256) {
                float f[8], w[8];
                load8(src + c, f);
                load8(weight + c, w);
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = f[e] * inv * w[e];
                store8(dst + c, f);
            }
        } else {
            for (long long c = lane; c < width; c += 32) Act<TO>::store(dst + c, Act<TX>::load(src + c) * inv * weight[c]);
        }
    }
}

// dx[r, c] = inv (g w - x inv^2 projected), projected = sum_c g w x / width   (lm_rms_dx, cpu_lm.py:84-104)
template <typename TG, typename TX, bool VEC>
__global__ void __launch_bounds__(kThreads)
rms_norm_dx_kernel(const TG* __restrict__ gradient, const TX* __restrict__ x, const float* __restrict__ weight,
                   const float* __restrict__ inverse, TX* __restrict__ dx, long long rows, long long width) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * kWarpsPerBlock;
    for (long long r = warp; r < rows; r += nwarps) {
        const TG* g = gradient + r * width;
        const TX* src = x + r * width;
        TX* dst = dx + r * width;
        float projected = 0.f;
        if (VEC) {
            for (long long c = lane * 8; c < width; c += 256) {
                float a[8], b[8], w[8];
                load8(g + c, a); load8(src + c, b); load8(weight + c, w);
#pragma unroll
                for (int e = 0; e < 8; ++e) projected = fmaf(a[e] * w[e], b[e], projected);
            }
        } else {
            for (long long c = lane; c < width; c += 32) projected = fmaf(Act<TG>::load(g + c) * weight[c], Act<TX>::load(src + c), projected);
        }
        projected = warp_sum(projected) / (float)width;
        const float inv = inverse[r];
        if (VEC) {
            for (long long c = lane * 8; c < width; c += 256) {
                float a[8], b[8], w[8];
                load8(g + c, a); load8(src + c, b); load8(weight + c, w);
#pragma unroll
                for (int e = 0; e < 8; ++e) a[e] = inv * (a[e] * w[e] - b[e] * inv * inv * projected);
                store8(dst + c, a);
            }
        } else {
            for (long long c = lane; c < width; c += 32)
                Act<TX>::store(dst + c, inv * (Act<TG>::load(g + c) * weight[c] - Act<TX>::load(src + c) * inv * inv * projected));
        }
    }
}

// partial[b, c] = sum over the rows of slab b of g[r, c] x[r, c] inverse[r]   (lm_rms_dw, one slab of rows per block)
template <typename TG, typename TX>
__global__ void __launch_bounds__(kThreads)
rms_norm_dw_partial_kernel(const TG* __restrict__ gradient, const TX* __restrict__ x, const float* __restrict__ inverse,
                           float* __restrict__ partial, long long rows, long long width) {
    const long long first = (long long)blockIdx.x * kSlabRows;
    const long long last = first + kSlabRows < rows ? first + kSlabRows : rows;
    for (long long c = threadIdx.x; c < width; c += kThreads) {
        float total = 0.f;
        for (long long r = first; r < last; ++r)
            total = fmaf(Act<TG>::load(gradient + r * width + c) * Act<TX>::load(x + r * width + c), inverse[r], total);
        partial[(long long)blockIdx.x * width + c] = total;
    }
}
__global__ void __launch_bounds__(kThreads)
sum_partials_kernel(const float* __restrict__ partial, float* __restrict__ out, long long slabs, long long width) {
    for (long long c = (long long)blockIdx.x * kThreads + threadIdx.x; c < width; c += (long long)gridDim.x * kThreads) {
        float total = 0.f;
        for (long long b = 0; b < slabs; ++b) total += partial[b * width + c];   // fixed order
        out[c] = total;
    }
}

// Rotation of every pair (2 i, 2 i + 1) of every head by (offset + t) theta^(-2 i / dim)   (lm_rope, cpu_lm.py:125-138)
template <typename T>
__global__ void __launch_bounds__(kThreads)
rope_kernel(const T* __restrict__ values, T* __restrict__ out, long long pairs, int time, int heads, int dim, float theta,
            int offset, int inverse) {
    const int half = dim / 2;
    const float step = -2.f * log2f(theta) / (float)dim;
    for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < pairs; i += (long long)gridDim.x * kThreads) {
        const int j = (int)(i % half);
        const long long t = (i / half / heads) % time;
        float angle = (float)(offset + t) * exp2f(step * (float)j);
        if (inverse) angle = -angle;
        float s, c;
        sincosf(angle, &s, &c);
        const float a = Act<T>::load(values + 2 * i), b = Act<T>::load(values + 2 * i + 1);
        Act<T>::store(out + 2 * i, a * c - b * s);
        Act<T>::store(out + 2 * i + 1, a * s + b * c);
    }
}

// out[i, :] = weight[ids[i], :]   (lm_embedding)
template <typename TO>
__global__ void __launch_bounds__(kThreads)
embedding_kernel(const float* __restrict__ weight, const long long* __restrict__ ids, TO* __restrict__ out, long long count,
                 long long width, long long vocab) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * kWarpsPerBlock;
    for (long long i = warp; i < count; i += nwarps) {
        const long long token = ids[i];
        const bool known = token >= 0 && token < vocab;     // an id outside the table reads nothing and gives a zero row
        for (long long c = lane; c < width; c += 32) Act<TO>::store(out + i * width + c, known ? weight[token * width + c] : 0.f);
    }
}

// d_weight[token[s], :] (+)= sum over the positions of segment s, in order, of gradient[position, :]
// (lm_embedding_backward: tokens sorted, each with the list of its positions)
template <typename TG>
__global__ void __launch_bounds__(kThreads)
embedding_backward_kernel(const TG* __restrict__ gradient, const long long* __restrict__ tokens, const long long* __restrict__ starts,
                          const long long* __restrict__ positions, float* __restrict__ d_weight, long long segments, long long width,
                          long long vocab, long long count) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * kWarpsPerBlock;
    for (long long s = warp; s < segments; s += nwarps) {
        const long long token = tokens[s];
        if (token < 0 || token >= vocab) continue;
        for (long long c = lane; c < width; c += 32) {
            float total = d_weight[token * width + c];
            for (long long at = starts[s]; at < starts[s + 1]; ++at) {
                const long long position = positions[at];
                if (position >= 0 && position < count) total += Act<TG>::load(gradient + position * width + c);
            }
            d_weight[token * width + c] = total;
        }
    }
}

bool known_dtype(int dtype) { return dtype == QMOE_F32 || dtype == QMOE_BF16; }

}  // namespace
}  // namespace qmoe

using namespace qmoe;

extern "C" int qmoe_rms_norm(uint64_t x, int32_t x_dtype, uint64_t weight, uint64_t out, int32_t out_dtype, uint64_t inverse,
                             int64_t rows, int64_t width, double eps, uint64_t stream_) {
    if (!x || !weight || !out || !inverse) return fail_arg("rms_norm: null address");
    if (rows <= 0 || width <= 0) return fail_arg("rms_norm: sizes must be positive");
    if (!known_dtype(x_dtype) || !known_dtype(out_dtype)) return fail_arg("rms_norm: dtype must be QMOE_F32 or QMOE_BF16");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_NORM, stream);
    const int grid = row_grid(rows);
    const float* w = (const float*)weight;
    float* inv = (float*)inverse;
    const bool vec = width % 8 == 0 && !((x | out | weight) & 31u);
#define QMOE_RMS_FORWARD(TX, TO)                                                                                               \
    do {                                                                                                                       \
        if (vec) rms_norm_kernel<TX, TO, true><<<grid, kThreads, 0, stream>>>((const TX*)x, w, (TO*)out, inv, rows, width, (float)eps);  \
        else rms_norm_kernel<TX, TO, false><<<grid, kThreads, 0, stream>>>((const TX*)x, w, (TO*)out, inv, rows, width, (float)eps);     \
    } while (0)
    if (x_dtype == QMOE_BF16 && out_dtype == QMOE_F32) QMOE_RMS_FORWARD(__nv_bfloat16, float);
    else if (x_dtype == QMOE_BF16) QMOE_RMS_FORWARD(__nv_bfloat16, __nv_bfloat16);
    else if (out_dtype == QMOE_F32) QMOE_RMS_FORWARD(float, float);
    else QMOE_RMS_FORWARD(float, __nv_bfloat16);
#undef QMOE_RMS_FORWARD
    QMOE_LAUNCH_CHECK("rms_norm_kernel");
    return 0;
}

extern "C" int64_t qmoe_rms_norm_partials(int64_t rows, int64_t width) {
    return rows > 0 && width > 0 ? ((rows + kSlabRows - 1) / kSlabRows) * width : 0;
}

extern "C" int qmoe_rms_norm_backward(uint64_t gradient, int32_t g_dtype, uint64_t x, int32_t x_dtype, uint64_t weight,
                                      uint64_t inverse, uint64_t dx, uint64_t d_weight, uint64_t partials, int64_t rows,
                                      int64_t width, uint64_t stream_) {
    if (!gradient || !x || !weight || !inverse || !dx || !d_weight || !partials) return fail_arg("rms_norm_backward: null address");
    if (rows <= 0 || width <= 0) return fail_arg("rms_norm_backward: sizes must be positive");
    if (!known_dtype(g_dtype) || !known_dtype(x_dtype)) return fail_arg("rms_norm_backward: dtype must be QMOE_F32 or QMOE_BF16");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_NORM, stream);
    const int grid = row_grid(rows);
    const long long slabs = (rows + kSlabRows - 1) / kSlabRows;
    const float* w = (const float*)weight;
    const float* inv = (const float*)inverse;
    float* part = (float*)partials;
    const bool vec = width % 8 == 0 && !((gradient | x | dx | weight) & 31u);
#define QMOE_RMS_BACKWARD(TG, TX)                                                                                              \
    do {                                                                                                                       \
        if (vec) rms_norm_dx_kernel<TG, TX, true><<<grid, kThreads, 0, stream>>>((const TG*)gradient, (const TX*)x, w, inv, (TX*)dx, rows, width);   \
        else rms_norm_dx_kernel<TG, TX, false><<<grid, kThreads, 0, stream>>>((const TG*)gradient, (const TX*)x, w, inv, (TX*)dx, rows, width);      \
        rms_norm_dw_partial_kernel<<<(unsigned)slabs, kThreads, 0, stream>>>((const TG*)gradient, (const TX*)x, inv, part, rows, width); \
    } while (0)
    if (g_dtype == QMOE_BF16 && x_dtype == QMOE_BF16) QMOE_RMS_BACKWARD(__nv_bfloat16, __nv_bfloat16);
    else if (g_dtype == QMOE_BF16) QMOE_RMS_BACKWARD(__nv_bfloat16, float);
    else if (x_dtype == QMOE_BF16) QMOE_RMS_BACKWARD(float, __nv_bfloat16);
    else QMOE_RMS_BACKWARD(float, float);
#undef QMOE_RMS_BACKWARD
    QMOE_LAUNCH_CHECK("rms_norm_dx_kernel");
    sum_partials_kernel<<<flat_grid(width), kThreads, 0, stream>>>(part, (float*)d_weight, slabs, width);
    QMOE_LAUNCH_CHECK("sum_partials_kernel");
    return 0;
}

extern "C" int qmoe_rope(uint64_t values, uint64_t out, int32_t dtype, int64_t batch, int64_t time, int32_t heads, int32_t dim,
                         double theta, int32_t offset, int32_t inverse, uint64_t stream_) {
    if (!values || !out) return fail_arg("rope: null address");
    if (batch <= 0 || time <= 0 || heads <= 0 || dim <= 0 || dim % 2 || theta <= 0) return fail_arg("rope: sizes must be positive, dim even, theta positive");
    if (!known_dtype(dtype)) return fail_arg("rope: dtype must be QMOE_F32 or QMOE_BF16");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_OTHER, stream);
    const long long pairs = batch * time * heads * (dim / 2);
    if (dtype == QMOE_BF16)
        rope_kernel<<<flat_grid(pairs), kThreads, 0, stream>>>((const __nv_bfloat16*)values, (__nv_bfloat16*)out, pairs, (int)time, heads, dim,
                                                               (float)theta, offset, inverse);
    else
        rope_kernel<<<flat_grid(pairs), kThreads, 0, stream>>>((const float*)values, (float*)out, pairs, (int)time, heads, dim, (float)theta,
                                                               offset, inverse);
    QMOE_LAUNCH_CHECK("rope_kernel");
    return 0;
}

extern "C" int qmoe_embedding(uint64_t weight, uint64_t ids, uint64_t out, int32_t out_dtype, int64_t count, int64_t width,
                              int64_t vocab, uint64_t stream_) {
    if (!weight || !ids || !out) return fail_arg("embedding: null address");
    if (count <= 0 || width <= 0 || vocab <= 0) return fail_arg("embedding: sizes must be positive");
    if (!known_dtype(out_dtype)) return fail_arg("embedding: dtype must be QMOE_F32 or QMOE_BF16");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_OTHER, stream);
    if (out_dtype == QMOE_BF16)
        embedding_kernel<<<row_grid(count), kThreads, 0, stream>>>((const float*)weight, (const long long*)ids, (__nv_bfloat16*)out, count, width, vocab);
    else
        embedding_kernel<<<row_grid(count), kThreads, 0, stream>>>((const float*)weight, (const long long*)ids, (float*)out, count, width, vocab);
    QMOE_LAUNCH_CHECK("embedding_kernel");
    return 0;
}

extern "C" int qmoe_embedding_backward(uint64_t gradient, int32_t g_dtype, uint64_t tokens, uint64_t starts, uint64_t positions,
                                       uint64_t d_weight, int64_t segments, int64_t count, int64_t width, int64_t vocab,
                                       uint64_t stream_) {
    if (!gradient || !tokens || !starts || !positions || !d_weight) return fail_arg("embedding_backward: null address");
    if (segments <= 0 || count <= 0 || width <= 0 || vocab <= 0) return fail_arg("embedding_backward: sizes must be positive");
    if (!known_dtype(g_dtype)) return fail_arg("embedding_backward: dtype must be QMOE_F32 or QMOE_BF16");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_OTHER, stream);
    if (g_dtype == QMOE_BF16)
        embedding_backward_kernel<<<row_grid(segments), kThreads, 0, stream>>>((const __nv_bfloat16*)gradient, (const long long*)tokens,
                                                                               (const long long*)starts, (const long long*)positions,
                                                                               (float*)d_weight, segments, width, vocab, count);
    else
        embedding_backward_kernel<<<row_grid(segments), kThreads, 0, stream>>>((const float*)gradient, (const long long*)tokens,
                                                                               (const long long*)starts, (const long long*)positions,
                                                                               (float*)d_weight, segments, width, vocab, count);
    QMOE_LAUNCH_CHECK("embedding_backward_kernel");
    return 0;
}
