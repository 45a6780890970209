// The step either side of the MoE layer inside a decoder block, fused into the layer's first read and last write:
//     out = x + MoE(rms_norm(x, w))
// (upstream: Block.__call__ src/qutai/lm/layers.py:430-437, rms_norm :88-96, kernels lm_rms / lm_rms_dx / lm_rms_dw
// src/qutai/backends/cuda/lm.cu:40-53, CPU statement src/qutai/backends/cpu_lm.py:84-117).  Upstream runs the norm as a
// kernel of its own that writes an fp32 copy of the activations, and the residual as another one that re-reads the
// layer's output; here
//   * a statistics pass leaves only 1 / rms per token (rms_inverse_kernel, reads x once);
//   * the dispatch gather normalises the row it copies (permute_norm_kernel) and the router product runs on the raw
//     x with the norm weight folded into the router weight and the row scale applied to the logits (scale_kernel);
//   * the weighted combine adds the residual row before its single rounding (combine_residual_kernel);
//   * in the backward the gather-sum that forms the gradient of the normalised input also applies the norm's
//     backward and adds the residual's gradient (unpermute_norm_backward_kernel), and leaves per-block partial sums
//     of the norm weight's gradient that are reduced in a fixed order (no floating-point atomics anywhere).
// One warp per token row, 16-byte accesses, like the kernels in permute.cu.
#include <initializer_list>

#include "common.cuh"

namespace qmoe {
namespace {

constexpr int kThreads = 256;
constexpr int kWarpsPerBlock = kThreads / 32;
constexpr long long kMaxFusedWidth = 4096;  // per-warp fp32 accumulators of the norm-weight gradient live in shared memory

__device__ __forceinline__ void st16(void* p, const uint4& v) { *reinterpret_cast<uint4*>(p) = v; }
__device__ __forceinline__ uint4 ld16_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
template <int N> __device__ __forceinline__ void load_f32(const float* p, float* f) {
#pragma unroll
    for (int i = 0; i < N; i += 4) {
        const float4 v = *reinterpret_cast<const float4*>(p + i);
        f[i] = v.x; f[i + 1] = v.y; f[i + 2] = v.z; f[i + 3] = v.w;
    }
}

// inverse[t] = 1 / sqrt(mean(x[t]^2) + eps)
template <typename T, bool VEC>
__global__ void __launch_bounds__(kThreads)
rms_inverse_kernel(const T* __restrict__ x, float* __restrict__ inverse, long long tokens, long long width, float eps) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * kWarpsPerBlock;
    for (long long t = warp; t < tokens; t += nwarps) {
        const T* src = x + t * width;
        float total = 0.f;
        if constexpr (VEC) {
            constexpr int N = Vec16<T>::N;
            for (int c = lane; c < (int)(width / N); c += 32) {
                float f[N];
                Vec16<T>::unpack(*reinterpret_cast<const uint4*>(src + (long long)c * N), f);
#pragma unroll
                for (int i = 0; i < N; ++i) total = fmaf(f[i], f[i], total);
            }
        } else {
            for (long long c = lane; c < width; c += 32) {
                const float v = Act<T>::load(src + c);
                total = fmaf(v, v, total);
            }
        }
        total = warp_sum(total);
        if (lane == 0) inverse[t] = rsqrtf(total / (float)width + eps);
    }
}

// out[r, c] = in[r, c] * (row_scale ? row_scale[r] : 1) * (col_scale ? col_scale[c] : 1), fp32, in place allowed
__global__ void __launch_bounds__(kThreads)
scale_kernel(const float* __restrict__ in, float* __restrict__ out, const float* __restrict__ row_scale,
             const float* __restrict__ col_scale, long long rows, long long cols) {
    const long long n = rows * cols;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const long long r = i / cols;
        float v = in[i];
        if (row_scale) v *= row_scale[r];
        if (col_scale) v *= col_scale[i - r * cols];
        out[i] = v;
    }
}

// dispatched[dest_row[t, s]] = round(x[t] * inverse[t] * w) for every slot, pads zero (the permute with the norm applied)
template <typename T, bool VEC, int KMAX>
__global__ void __launch_bounds__(kThreads)
permute_norm_kernel(const T* __restrict__ x, const float* __restrict__ inverse, const float* __restrict__ weight,
                    T* __restrict__ out, const int* __restrict__ dest_row, const int* __restrict__ row_source,
                    const int* __restrict__ meta, long long tokens, int k, long long width) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * kWarpsPerBlock + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * kWarpsPerBlock;
    for (long long t = warp; t < tokens; t += nwarps) {
        long long rows[KMAX];
#pragma unroll
        for (int s = 0; s < KMAX; ++s) rows[s] = s < k ? dest_row[t * k + s] : 0;
        const T* src = x + t * width;
        const float inv = inverse[t];
        if constexpr (VEC) {
            constexpr int N = Vec16<T>::N;
            for (int c = lane; c < (int)(width / N); c += 32) {
                float f[N], w[N];
                Vec16<T>::unpack(ld16_stream(src + (long long)c * N), f);
                load_f32<N>(weight + (long long)c * N, w);
#pragma unroll
                for (int i = 0; i < N; ++i) f[i] = f[i] * inv * w[i];
                const uint4 v = Vec16<T>::pack(f);
#pragma unroll
                for (int s = 0; s < KMAX; ++s)
                    if (s < k) st16(out + rows[s] * width + (long long)c * N, v);
            }
        } else {
            for (long long c = lane; c < width; c += 32) {
                T v;
                Act<T>::store(&v, Act<T>::load(src + c) * inv * weight[c]);
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

// out[t] = round(residual[t] + sum_s w[t, s] * y[dest_row[t, s]]): fp32 sum, one rounding
template <typename T, bool VEC, int KMAX>
__global__ void __launch_bounds__(kThreads)
combine_residual_kernel(const T* __restrict__ y, const float* __restrict__ gate_w, const int* __restrict__ dest_row,
                        const T* __restrict__ residual, T* __restrict__ out, long long tokens, int k, long long width) {
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
        const T* res = residual + t * width;
        if constexpr (VEC) {
            constexpr int N = Vec16<T>::N;
            for (int c = lane; c < (int)(width / N); c += 32) {
                uint4 v[KMAX];
#pragma unroll
                for (int s = 0; s < KMAX; ++s)
                    if (s < k) v[s] = ld16_stream(y + (long long)rows[s] * width + (long long)c * N);
                float acc[N], base[N];
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
                Vec16<T>::unpack(ld16_stream(res + (long long)c * N), base);
#pragma unroll
                for (int i = 0; i < N; ++i) acc[i] += base[i];
                st16(dst + (long long)c * N, Vec16<T>::pack(acc));
            }
        } else {
            for (long long c = lane; c < width; c += 32) {
                float acc = 0.f;
                for (int s = 0; s < k; ++s) acc = fmaf(w[s], Act<T>::load(y + (long long)rows[s] * width + c), acc);
                Act<T>::store(dst + c, acc + Act<T>::load(res + c));
            }
        }
    }
}

// The gather-sum of the layer's input gradient with the norm's backward and the residual's gradient folded in.  With
// d_n[t] = sum_s d_dispatched[dest_row[t, s]] + extra[t] (the gradient of the normalised input):
//     projected = mean_j(d_n[j] * w[j] * x[t, j])
//     dx[t, j]  = round(grad_out[t, j] + inverse * (d_n[j] * w[j] - x[t, j] * inverse^2 * projected))
//     dw[j]    += d_n[j] * x[t, j] * inverse
// Two passes over the token's rows (the second finds them in L2): the first forms `projected`, the second writes dx
// and adds this row's share of dw into the warp's shared-memory accumulators.  At the end the block adds its warps'
// accumulators in warp order and writes one row of `partials` [blocks, width].
template <typename T, bool VEC, int KMAX>
__global__ void __launch_bounds__(kThreads)
unpermute_norm_backward_kernel(const T* __restrict__ dxd, const float* __restrict__ extra, int extra_row_scaled,
                               const int* __restrict__ dest_row, const T* __restrict__ x, const float* __restrict__ inverse,
                               const float* __restrict__ weight, const T* __restrict__ grad_out, T* __restrict__ dx,
                               float* __restrict__ partials, long long tokens, int k, long long width) {
    extern __shared__ float s_dw[];  // [warps][width]
    const int lane = threadIdx.x & 31, warp_in_block = threadIdx.x >> 5;
    const long long warp = (long long)blockIdx.x * kWarpsPerBlock + warp_in_block;
    const long long nwarps = (long long)gridDim.x * kWarpsPerBlock;
    float* mine = s_dw + (long long)warp_in_block * width;
    for (long long c = lane; c < width; c += 32) mine[c] = 0.f;
    __syncwarp();
    for (long long t = warp; t < tokens; t += nwarps) {
        int rows[KMAX];
#pragma unroll
        for (int s = 0; s < KMAX; ++s) rows[s] = s < k ? dest_row[t * k + s] : 0;
        const T* xs = x + t * width;
        const float inv = inverse[t];
        // extra_row_scaled: `extra` holds inverse[t] times the addend (the router's product ran on row-scaled logit gradients)
        const float extra_scale = extra_row_scaled ? 1.f / inv : 1.f;
        float projected = 0.f;
        if constexpr (VEC) {
            constexpr int N = Vec16<T>::N;
            const int chunks = (int)(width / N);
            auto gather = [&](int c, float* acc) {  // d_n of 16 bytes' worth of columns
                uint4 v[KMAX];
#pragma unroll
                for (int s = 0; s < KMAX; ++s)
                    if (s < k) v[s] = *reinterpret_cast<const uint4*>(dxd + (long long)rows[s] * width + (long long)c * N);
                if (extra) {
                    load_f32<N>(extra + t * width + (long long)c * N, acc);
#pragma unroll
                    for (int i = 0; i < N; ++i) acc[i] *= extra_scale;
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
            };
            for (int c = lane; c < chunks; c += 32) {
                float dn[N], fx[N], w[N];
                gather(c, dn);
                Vec16<T>::unpack(*reinterpret_cast<const uint4*>(xs + (long long)c * N), fx);
                load_f32<N>(weight + (long long)c * N, w);
#pragma unroll
                for (int i = 0; i < N; ++i) projected = fmaf(dn[i] * w[i], fx[i], projected);
            }
            projected = warp_sum(projected) / (float)width;
            const float pull = inv * inv * projected;
            for (int c = lane; c < chunks; c += 32) {
                float dn[N], fx[N], w[N], g[N], o[N];
                gather(c, dn);
                Vec16<T>::unpack(*reinterpret_cast<const uint4*>(xs + (long long)c * N), fx);
                load_f32<N>(weight + (long long)c * N, w);
                Vec16<T>::unpack(ld16_stream(grad_out + t * width + (long long)c * N), g);
#pragma unroll
                for (int i = 0; i < N; ++i) {
                    o[i] = g[i] + inv * (dn[i] * w[i] - fx[i] * pull);
                    // column c * N + i is kept at i * chunks + c: the 32 lanes of a warp touch consecutive words
                    mine[(long long)i * chunks + c] += dn[i] * fx[i] * inv;
                }
                st16(dx + t * width + (long long)c * N, Vec16<T>::pack(o));
            }
        } else {
            auto gather = [&](long long c) {
                float acc = extra ? extra[t * width + c] * extra_scale : 0.f;
                for (int s = 0; s < k; ++s) acc += Act<T>::load(dxd + (long long)rows[s] * width + c);
                return acc;
            };
            for (long long c = lane; c < width; c += 32) projected = fmaf(gather(c) * weight[c], Act<T>::load(xs + c), projected);
            projected = warp_sum(projected) / (float)width;
            const float pull = inv * inv * projected;
            for (long long c = lane; c < width; c += 32) {
                const float dn = gather(c), fx = Act<T>::load(xs + c);
                Act<T>::store(dx + t * width + c, Act<T>::load(grad_out + t * width + c) + inv * (dn * weight[c] - fx * pull));
                mine[c] += dn * fx * inv;
            }
        }
    }
    __syncthreads();
    for (long long at = threadIdx.x; at < width; at += kThreads) {
        float total = 0.f;
#pragma unroll
        for (int w = 0; w < kWarpsPerBlock; ++w) total += s_dw[(long long)w * width + at];
        long long column = at;
        if constexpr (VEC) {  // undo the interleaved placement of the accumulators
            constexpr int N = Vec16<T>::N;
            const long long chunks = width / N;
            column = (at % chunks) * N + at / chunks;
        }
        partials[(long long)blockIdx.x * width + column] = total;
    }
}

bool aligned16(uint64_t p) { return (p & 15u) == 0; }
template <typename T>
bool can_vec(long long width, std::initializer_list<uint64_t> ptrs) {
    if ((width * (long long)sizeof(T)) % 16 || width % 4) return false;
    for (uint64_t p : ptrs)
        if (p && !aligned16(p)) return false;
    return true;
}
int grid_for_rows(long long rows, int blocks_per_sm) {
    long long blocks = (rows + kWarpsPerBlock - 1) / kWarpsPerBlock;
    const long long cap = (long long)sm_count() * blocks_per_sm;
    if (blocks > cap) blocks = cap;
    return (int)(blocks < 1 ? 1 : blocks);
}
int check_dtype(int dtype) {
    if (dtype != QMOE_F32 && dtype != QMOE_BF16) return fail_arg("dtype must be QMOE_F32 or QMOE_BF16 (got %d)", dtype);
    return 0;
}
// blocks of the backward kernel: as many per SM as their shared-memory accumulators (8 warps x width floats) allow
int backward_grid(long long tokens, long long width) {
    const long long per_block = (long long)kWarpsPerBlock * width * (long long)sizeof(float);
    long long per_sm = (216ll * 1024) / (per_block > 0 ? per_block : 1);
    per_sm = per_sm < 1 ? 1 : per_sm > 8 ? 8 : per_sm;
    return grid_for_rows(tokens, (int)per_sm);
}

// out[c] = sum over rows of partials[row, c] in a fixed order: 32 strided partial sums per column, then those 32 in order
__global__ void __launch_bounds__(1024)
reduce_rows_kernel(const float* __restrict__ partials, float* __restrict__ out, int rows, long long width) {
    __shared__ float s_part[32][33];
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const long long c = (long long)blockIdx.x * 32 + tx;
    float total = 0.f;
    if (c < width)
        for (int r = ty; r < rows; r += 32) total += partials[(long long)r * width + c];
    s_part[ty][tx] = total;
    __syncthreads();
    if (ty == 0 && c < width) {
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 32; ++i) sum += s_part[i][tx];
        out[c] = sum;
    }
}

}  // namespace
}  // namespace qmoe

using namespace qmoe;

#define BY_K(KERNEL, T, V, ...)                                                   \
    do {                                                                          \
        if (r->top_k <= 1) KERNEL<T, V, 1> __VA_ARGS__;                            \
        else if (r->top_k <= 2) KERNEL<T, V, 2> __VA_ARGS__;                       \
        else if (r->top_k <= 4) KERNEL<T, V, 4> __VA_ARGS__;                       \
        else if (r->top_k <= 6) KERNEL<T, V, 6> __VA_ARGS__;                       \
        else KERNEL<T, V, 8> __VA_ARGS__;                                          \
    } while (0)
#define BY_TYPE(KERNEL, ...)                                                       \
    do {                                                                          \
        if (dtype == QMOE_BF16) { if (vec) BY_K(KERNEL, __nv_bfloat16, true, __VA_ARGS__); else BY_K(KERNEL, __nv_bfloat16, false, __VA_ARGS__); } \
        else { if (vec) BY_K(KERNEL, float, true, __VA_ARGS__); else BY_K(KERNEL, float, false, __VA_ARGS__); }                                   \
    } while (0)

extern "C" int qmoe_rms_inverse(uint64_t x, int32_t dtype, uint64_t inverse, int64_t tokens, int64_t width, double eps,
                                uint64_t stream_) {
    if (int rc = check_dtype(dtype)) return rc;
    if (!x || !inverse || tokens <= 0 || width <= 0) return fail_arg("rms_inverse: null address or non-positive size");
    if (!(eps >= 0)) return fail_arg("rms_inverse: eps must not be negative");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_NORM, stream);
    const int grid = grid_for_rows(tokens, 8);
    if (dtype == QMOE_BF16) {
        if (can_vec<__nv_bfloat16>(width, {x}))
            rms_inverse_kernel<__nv_bfloat16, true><<<grid, kThreads, 0, stream>>>((const __nv_bfloat16*)x, (float*)inverse, tokens, width, (float)eps);
        else
            rms_inverse_kernel<__nv_bfloat16, false><<<grid, kThreads, 0, stream>>>((const __nv_bfloat16*)x, (float*)inverse, tokens, width, (float)eps);
    } else {
        if (can_vec<float>(width, {x}))
            rms_inverse_kernel<float, true><<<grid, kThreads, 0, stream>>>((const float*)x, (float*)inverse, tokens, width, (float)eps);
        else
            rms_inverse_kernel<float, false><<<grid, kThreads, 0, stream>>>((const float*)x, (float*)inverse, tokens, width, (float)eps);
    }
    QMOE_LAUNCH_CHECK("rms_inverse_kernel");
    return 0;
}

extern "C" int qmoe_scale_f32(uint64_t in, uint64_t out, uint64_t row_scale, uint64_t col_scale, int64_t rows, int64_t cols,
                              uint64_t stream_) {
    if (!in || !out || rows <= 0 || cols <= 0) return fail_arg("scale_f32: null address or non-positive size");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_NORM, stream);
    const long long n = rows * cols;
    const long long blocks = (n + kThreads - 1) / kThreads, cap = (long long)sm_count() * 8;
    scale_kernel<<<(int)(blocks < cap ? blocks : cap), kThreads, 0, stream>>>((const float*)in, (float*)out, (const float*)row_scale,
                                                                             (const float*)col_scale, rows, cols);
    QMOE_LAUNCH_CHECK("scale_kernel");
    return 0;
}

extern "C" int qmoe_permute_norm(const qmoe_route_t* r, uint64_t x, uint64_t inverse, uint64_t norm_weight, uint64_t out,
                                 int32_t dtype, int64_t width, uint64_t stream_) {
    if (int rc = route_check(r)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (!x || !inverse || !norm_weight || !out || width <= 0) return fail_arg("permute_norm: null address or non-positive width");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_PERMUTE, stream);
    const bool vec = dtype == QMOE_BF16 ? can_vec<__nv_bfloat16>(width, {x, out, norm_weight}) : can_vec<float>(width, {x, out, norm_weight});
    const int grid = grid_for_rows(r->tokens > (long long)r->experts * 64 ? r->tokens : (long long)r->experts * 64, 8);
#define ARGS(T) <<<grid, kThreads, 0, stream>>>((const T*)x, (const float*)inverse, (const float*)norm_weight, (T*)out,       \
        (const int*)r->dest_row, (const int*)r->row_source, (const int*)r->meta, (long long)r->tokens, r->top_k, (long long)width)
    if (dtype == QMOE_BF16) { if (vec) BY_K(permute_norm_kernel, __nv_bfloat16, true, ARGS(__nv_bfloat16)); else BY_K(permute_norm_kernel, __nv_bfloat16, false, ARGS(__nv_bfloat16)); }
    else { if (vec) BY_K(permute_norm_kernel, float, true, ARGS(float)); else BY_K(permute_norm_kernel, float, false, ARGS(float)); }
#undef ARGS
    QMOE_LAUNCH_CHECK("permute_norm_kernel");
    return 0;
}

extern "C" int qmoe_combine_residual(const qmoe_route_t* r, uint64_t y, uint64_t residual, uint64_t out, int32_t dtype,
                                     int64_t width, uint64_t stream_) {
    if (int rc = route_check(r)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (!y || !residual || !out || width <= 0) return fail_arg("combine_residual: null address or non-positive width");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_COMBINE, stream);
    const bool vec = dtype == QMOE_BF16 ? can_vec<__nv_bfloat16>(width, {y, residual, out}) : can_vec<float>(width, {y, residual, out});
    const int grid = grid_for_rows(r->tokens, 8);
#define ARGS(T) <<<grid, kThreads, 0, stream>>>((const T*)y, (const float*)r->gate_weights, (const int*)r->dest_row,           \
        (const T*)residual, (T*)out, (long long)r->tokens, r->top_k, (long long)width)
    if (dtype == QMOE_BF16) { if (vec) BY_K(combine_residual_kernel, __nv_bfloat16, true, ARGS(__nv_bfloat16)); else BY_K(combine_residual_kernel, __nv_bfloat16, false, ARGS(__nv_bfloat16)); }
    else { if (vec) BY_K(combine_residual_kernel, float, true, ARGS(float)); else BY_K(combine_residual_kernel, float, false, ARGS(float)); }
#undef ARGS
    QMOE_LAUNCH_CHECK("combine_residual_kernel");
    return 0;
}

extern "C" int64_t qmoe_norm_backward_partials(int64_t tokens, int64_t width) {
    if (tokens <= 0 || width <= 0) return 0;
    return (int64_t)backward_grid(tokens, width) * width;
}

extern "C" int qmoe_unpermute_norm_backward(const qmoe_route_t* r, uint64_t d_dispatched, uint64_t extra_f32,
                                            int32_t extra_row_scaled, uint64_t x, uint64_t inverse, uint64_t norm_weight,
                                            uint64_t grad_out, uint64_t dx, uint64_t d_norm_weight, uint64_t partials,
                                            int32_t dtype, int64_t width, uint64_t stream_) {
    if (int rc = route_check(r)) return rc;
    if (int rc = check_dtype(dtype)) return rc;
    if (!d_dispatched || !x || !inverse || !norm_weight || !grad_out || !dx || !d_norm_weight || !partials || width <= 0)
        return fail_arg("unpermute_norm_backward: null address or non-positive width");
    if (width > kMaxFusedWidth) {
        set_error("unpermute_norm_backward: width %lld exceeds the fused kernel's %lld", (long long)width, kMaxFusedWidth);
        return QMOE_ERR_UNSUPPORTED;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_UNPERMUTE, stream);
    const bool vec = dtype == QMOE_BF16 ? can_vec<__nv_bfloat16>(width, {d_dispatched, extra_f32, x, norm_weight, grad_out, dx})
                                        : can_vec<float>(width, {d_dispatched, extra_f32, x, norm_weight, grad_out, dx});
    const int grid = backward_grid(r->tokens, width);
    const size_t smem = (size_t)kWarpsPerBlock * width * sizeof(float);
#define LAUNCH(T, V, K)                                                                                                        \
    do {                                                                                                                       \
        auto kernel = unpermute_norm_backward_kernel<T, V, K>;                                                                 \
        if (smem > 48 * 1024) QMOE_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); \
        kernel<<<grid, kThreads, smem, stream>>>((const T*)d_dispatched, (const float*)extra_f32, extra_row_scaled,            \
            (const int*)r->dest_row,                                                                                           \
            (const T*)x, (const float*)inverse, (const float*)norm_weight, (const T*)grad_out, (T*)dx, (float*)partials,      \
            (long long)r->tokens, r->top_k, (long long)width);                                                                 \
    } while (0)
#define LAUNCH_K(T, V)                                                     \
    do {                                                                   \
        if (r->top_k <= 1) LAUNCH(T, V, 1); else if (r->top_k <= 2) LAUNCH(T, V, 2); else if (r->top_k <= 4) LAUNCH(T, V, 4); \
        else if (r->top_k <= 6) LAUNCH(T, V, 6); else LAUNCH(T, V, 8);     \
    } while (0)
    if (dtype == QMOE_BF16) { if (vec) LAUNCH_K(__nv_bfloat16, true); else LAUNCH_K(__nv_bfloat16, false); }
    else { if (vec) LAUNCH_K(float, true); else LAUNCH_K(float, false); }
#undef LAUNCH_K
#undef LAUNCH
    QMOE_LAUNCH_CHECK("unpermute_norm_backward_kernel");
    reduce_rows_kernel<<<(int)((width + 31) / 32), 1024, 0, stream>>>((const float*)partials, (float*)d_norm_weight, grid, width);
    QMOE_LAUNCH_CHECK("reduce_rows_kernel");
    return 0;
}
