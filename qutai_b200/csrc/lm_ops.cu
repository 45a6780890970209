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
constexpr int kSlabRows = 32;          // rows of one block of the norm weight's gradient

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

// eight elements as they lie in memory, converted when they are used (keeps many loads in flight in few registers)
template <typename T> struct Raw8;
template <> struct Raw8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float* p) { a = *reinterpret_cast<const float4*>(p); b = *reinterpret_cast<const float4*>(p + 4); }
    __device__ __forceinline__ void unpack(float* f) const { f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w; }
};
template <> struct Raw8<__nv_bfloat16> {
    uint4 v;
    __device__ __forceinline__ void load(const __nv_bfloat16* p) { v = *reinterpret_cast<const uint4*>(p); }
    __device__ __forceinline__ void unpack(float* f) const { Vec16<__nv_bfloat16>::unpack(v, f); }
};

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
template <typename TG, typename TX, bool VEC>
__global__ void __launch_bounds__(kThreads)
rms_norm_dw_partial_kernel(const TG* __restrict__ gradient, const TX* __restrict__ x, const float* __restrict__ inverse,
                           float* __restrict__ partial, long long rows, long long width) {
    const long long first = (long long)blockIdx.x * kSlabRows;
    const long long last = first + kSlabRows < rows ? first + kSlabRows : rows;
    if (VEC) {   // a thread owns eight neighbouring columns; the rows are added in order, four of them in flight
        for (long long c = (long long)threadIdx.x * 8; c < width; c += 8ll * kThreads) {
            float total[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            for (long long r0 = first; r0 < last; r0 += 4) {
                float g[4][8], v[4][8], inv[4];
#pragma unroll
                for (int u = 0; u < 4; ++u) {
                    const long long r = r0 + u < last ? r0 + u : last - 1;
                    load8(gradient + r * width + c, g[u]);
                    load8(x + r * width + c, v[u]);
                    inv[u] = r0 + u < last ? inverse[r] : 0.f;
                }
#pragma unroll
                for (int u = 0; u < 4; ++u)
#pragma unroll
                    for (int j = 0; j < 8; ++j) total[j] = fmaf(g[u][j] * v[u][j], inv[u], total[j]);
            }
            store8(partial + (long long)blockIdx.x * width + c, total);
        }
        return;
    }
    for (long long c = threadIdx.x; c < width; c += kThreads) {
        float total = 0.f;
        for (long long r = first; r < last; ++r)
            total = fmaf(Act<TG>::load(gradient + r * width + c) * Act<TX>::load(x + r * width + c), inverse[r], total);
        partial[(long long)blockIdx.x * width + c] = total;
    }
}
// out[c] = sum over the slabs, in order.  A block owns 32 columns; its eight warps take the slabs b = w, w + 8, ... and
// their sums are added in the order of w: the same tree on every run.
__global__ void __launch_bounds__(kThreads)
sum_partials_kernel(const float* __restrict__ partial, float* __restrict__ out, long long slabs, long long width) {
    __shared__ float part[kWarpsPerBlock][32];
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
    for (long long c0 = (long long)blockIdx.x * 32; c0 < width; c0 += (long long)gridDim.x * 32) {
        const long long c = c0 + lane;
        float total = 0.f;
        if (c < width)
            for (long long b = w; b < slabs; b += kWarpsPerBlock) total += partial[b * width + c];
        part[w][lane] = total;
        __syncthreads();
        if (w == 0 && c < width) {
            float sum = part[0][lane];
#pragma unroll
            for (int i = 1; i < kWarpsPerBlock; ++i) sum += part[i][lane];
            out[c] = sum;
        }
        __syncthreads();
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
// The same rotation with the angles of a position computed once for all its heads: a thread owns (sequence, position,
// four neighbouring pairs = eight elements) and walks the heads.  dim a multiple of 8, rows on 32-byte boundaries.
template <typename T>
__global__ void __launch_bounds__(kThreads)
rope_heads_kernel(const T* __restrict__ values, T* __restrict__ out, long long positions, int time, int heads, int dim, float theta,
                  int offset, int inverse) {
    const int groups = dim / 8;
    const float step = -2.f * log2f(theta) / (float)dim;
    for (long long i = (long long)blockIdx.x * kThreads + threadIdx.x; i < positions * groups; i += (long long)gridDim.x * kThreads) {
        const int group = (int)(i % groups);
        const long long position = i / groups, t = position % time;
        float s[4], c[4];
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            float angle = (float)(offset + t) * exp2f(step * (float)(4 * group + q));
            if (inverse) angle = -angle;
            sincosf(angle, &s[q], &c[q]);
        }
        const long long base = position * heads * dim + 8 * group;
        for (int h = 0; h < heads; ++h) {
            float f[8], r[8];
            load8(values + base + (long long)h * dim, f);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                r[2 * q] = f[2 * q] * c[q] - f[2 * q + 1] * s[q];
                r[2 * q + 1] = f[2 * q] * s[q] + f[2 * q + 1] * c[q];
            }
            store8(out + base + (long long)h * dim, r);
        }
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
template <typename TG, bool VEC>
__global__ void __launch_bounds__(kThreads)
embedding_backward_kernel(const TG* __restrict__ gradient, const long long* __restrict__ tokens, const long long* __restrict__ starts,
                          const long long* __restrict__ positions, float* __restrict__ d_weight, long long segments, long long width,
                          long long vocab, long long count, int parts) {
    // A warp owns (segment, part): columns [part * span, (part + 1) * span) of the token's row.
    // A frequent token has thousands of positions (Zipf-distributed ids put a third of a batch on one token); its
    // row is walked by `parts` warps side by side, each adding the positions in the order given, four rows in flight.
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5), nwarps = (long long)gridDim.x * kWarpsPerBlock;
    const long long span = VEC ? 256 : width;   // the launch gives parts = ceil(width / 256) in the vector form, else 1
    for (long long item = warp; item < segments * parts; item += nwarps) {
        const long long s = item / parts, part = item - s * parts;
        const long long token = tokens[s];
        if (token < 0 || token >= vocab) continue;
        const long long begin = starts[s], end = starts[s + 1];
        const long long c_begin = part * span, c_end = c_begin + span < width ? c_begin + span : width;
        float* row = d_weight + token * width;
        if (VEC) {
            for (long long c = c_begin + lane * 8; c < c_end; c += 256) {
                float total[8];
                load8(row + c, total);
                long long at = begin;
                constexpr int kFlight = sizeof(TG) == 2 ? 16 : 8;     // rows in flight: 16 bytes (bf16) or 32 (fp32) per lane each
                for (; at + kFlight <= end; at += kFlight) {
                    Raw8<TG> raw[kFlight];
                    bool in[kFlight];
#pragma unroll
                    for (int u = 0; u < kFlight; ++u) {
                        const long long position = positions[at + u];
                        in[u] = position >= 0 && position < count;
                        if (in[u]) raw[u].load(gradient + position * width + c);
                    }
#pragma unroll
                    for (int u = 0; u < kFlight; ++u)
                        if (in[u]) {
                            float f[8];
                            raw[u].unpack(f);
#pragma unroll
                            for (int j = 0; j < 8; ++j) total[j] += f[j];
                        }
                }
                for (; at < end; ++at) {
                    const long long position = positions[at];
                    if (position < 0 || position >= count) continue;
                    float f[8];
                    load8(gradient + position * width + c, f);
#pragma unroll
                    for (int j = 0; j < 8; ++j) total[j] += f[j];
                }
                store8(row + c, total);
            }
        } else {
            for (long long c = c_begin + lane; c < c_end; c += 32) {
                float total = row[c];
                for (long long at = begin; at < end; ++at) {
                    const long long position = positions[at];
                    if (position >= 0 && position < count) total += Act<TG>::load(gradient + position * width + c);
                }
                row[c] = total;
            }
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
    const bool vec = width % 8 == 0 && !((gradient | x | dx | weight | partials) & 31u);
#define QMOE_RMS_BACKWARD(TG, TX)                                                                                              \
    do {                                                                                                                       \
        if (vec) rms_norm_dx_kernel<TG, TX, true><<<grid, kThreads, 0, stream>>>((const TG*)gradient, (const TX*)x, w, inv, (TX*)dx, rows, width);   \
        else rms_norm_dx_kernel<TG, TX, false><<<grid, kThreads, 0, stream>>>((const TG*)gradient, (const TX*)x, w, inv, (TX*)dx, rows, width);      \
        if (vec) rms_norm_dw_partial_kernel<TG, TX, true><<<(unsigned)slabs, kThreads, 0, stream>>>((const TG*)gradient, (const TX*)x, inv, part, rows, width); \
        else rms_norm_dw_partial_kernel<TG, TX, false><<<(unsigned)slabs, kThreads, 0, stream>>>((const TG*)gradient, (const TX*)x, inv, part, rows, width); \
    } while (0)
    if (g_dtype == QMOE_BF16 && x_dtype == QMOE_BF16) QMOE_RMS_BACKWARD(__nv_bfloat16, __nv_bfloat16);
    else if (g_dtype == QMOE_BF16) QMOE_RMS_BACKWARD(__nv_bfloat16, float);
    else if (x_dtype == QMOE_BF16) QMOE_RMS_BACKWARD(float, __nv_bfloat16);
    else QMOE_RMS_BACKWARD(float, float);
#undef QMOE_RMS_BACKWARD
    QMOE_LAUNCH_CHECK("rms_norm_dx_kernel");
    sum_partials_kernel<<<(unsigned)((width + 31) / 32), kThreads, 0, stream>>>(part, (float*)d_weight, slabs, width);
    QMOE_LAUNCH_CHECK("sum_partials_kernel");
    return 0;
}

extern "C" int qmoe_rope(uint64_t values, uint64_t out, int32_t dtype, int64_t batch, int64_t time, int32_t heads, int32_t dim,
                         double theta, int32_t offset, int32_t inverse, uint64_t stream_) {
    if (!values || !out) return fail_arg("rope: null address");
    if (batch <= 0 || time <= 0 || heads <= 0 || dim <= 0 || dim % 2 || theta <= 0) return fail_arg("rope: sizes must be positive, dim even, theta positive");
    if (!known_dtype(dtype)) return fail_arg("rope: dtype must be QMOE_F32 or QMOE_BF16");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_ELEMENTWISE, stream);
    const long long pairs = batch * time * heads * (dim / 2), positions = batch * time;
    const bool by_position = dim % 8 == 0 && !((values | out) & 31u);
    if (by_position && dtype == QMOE_BF16)
        rope_heads_kernel<<<flat_grid(positions * (dim / 8)), kThreads, 0, stream>>>((const __nv_bfloat16*)values, (__nv_bfloat16*)out, positions,
                                                                                     (int)time, heads, dim, (float)theta, offset, inverse);
    else if (by_position)
        rope_heads_kernel<<<flat_grid(positions * (dim / 8)), kThreads, 0, stream>>>((const float*)values, (float*)out, positions, (int)time,
                                                                                     heads, dim, (float)theta, offset, inverse);
    else if (dtype == QMOE_BF16)
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
    TimedScope timed(KC_ELEMENTWISE, stream);
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
    TimedScope timed(KC_ELEMENTWISE, stream);
    // vector form: rows of 8-element pieces on 32-byte boundaries; spans of 256 columns per warp
    const bool vec = width % 8 == 0 && !((gradient | d_weight) & 31u);
    const int parts = vec ? (int)((width + 255) / 256) : 1;
    const int grid = row_grid(segments * parts);
#define QMOE_EMBEDDING_BACKWARD(TG, VEC)                                                                                              \
    embedding_backward_kernel<TG, VEC><<<grid, kThreads, 0, stream>>>((const TG*)gradient, (const long long*)tokens, (const long long*)starts, \
                                                                      (const long long*)positions, (float*)d_weight, segments, width, vocab, \
                                                                      count, parts)
    if (g_dtype == QMOE_BF16) {
        if (vec) QMOE_EMBEDDING_BACKWARD(__nv_bfloat16, true); else QMOE_EMBEDDING_BACKWARD(__nv_bfloat16, false);
    } else {
        if (vec) QMOE_EMBEDDING_BACKWARD(float, true); else QMOE_EMBEDDING_BACKWARD(float, false);
    }
#undef QMOE_EMBEDDING_BACKWARD
    QMOE_LAUNCH_CHECK("embedding_backward_kernel");
    return 0;
}
