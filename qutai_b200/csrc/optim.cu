// The optimizer step for the layer's parameters: AdamW over many tensors in one launch, with the bf16
// operand copies of the expert weights refreshed in the same pass, and the global gradient-norm clip.
// Upstream launches one element-wise kernel per parameter tensor (src/qutai/nn/optimizers.py:136-153,
// src/qutai/backends/cuda.py:449-452, src/qutai/backends/cuda/tensor.cu:101-104) and three per tensor
// for the clip (src/qutai/nn/optimizers.py:19-31, src/qutai/backends/cuda.py:425-437, :150-154).
//
// All kernels are HBM-bound streams: AdamW reads p, g, m, v and writes p, m, v (28 bytes per element,
// 30 with the bf16 copy); the clip reads every gradient once and, when the norm is above the limit,
// reads and writes it once more.
#include "common.cuh"

namespace qmoe {

namespace {

constexpr int kOptimThreads = 256;
constexpr int kChunk = 4096;  // elements per work unit: 256 threads x 4 float4

struct Item {  // = qmoe_optim_item_t
    float* values;
    float* grad;
    float* m;
    float* v;
    __nv_bfloat16* shadow;
    long long size;
    long long first_chunk;
    float c1, c2;
};
static_assert(sizeof(Item) == sizeof(qmoe_optim_item_t), "the table layout is part of the C ABI");

// the item whose chunk range holds `chunk`: the last one with first_chunk <= chunk
__device__ __forceinline__ int find_item(const Item* items, int count, long long chunk) {
    int lo = 0, hi = count;
    while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (items[mid].first_chunk <= chunk) lo = mid; else hi = mid;
    }
    return lo;
}

// One element, in the operation order of the upstream kernel (fp32 throughout).
__device__ __forceinline__ void adamw_element(float& p, float g, float& m, float& v, float lr, float b1, float b2,
                                              float c1, float c2, float eps, float decay) {
    m = b1 * m + (1.f - b1) * g;
    v = b2 * v + (1.f - b2) * g * g;
    p = p * (1.f - lr * decay) - lr * __fdiv_rn(m, c1) / (__fsqrt_rn(__fdiv_rn(v, c2)) + eps);
}

__global__ void __launch_bounds__(kOptimThreads)
adamw_multi_kernel(const Item* __restrict__ items, int count, long long total_chunks, float lr, float b1, float b2,
                   float eps, float decay) {
    for (long long chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
        const Item it = items[find_item(items, count, chunk)];
        const long long base = (chunk - it.first_chunk) * kChunk;
        const bool vec = ((((uintptr_t)it.values | (uintptr_t)it.grad | (uintptr_t)it.m | (uintptr_t)it.v) & 15u) == 0) &&
                         (!it.shadow || ((uintptr_t)it.shadow & 7u) == 0);
#pragma unroll
        for (int r = 0; r < kChunk / (kOptimThreads * 4); ++r) {
            const long long i = base + ((long long)r * kOptimThreads + threadIdx.x) * 4;
            if (i >= it.size) break;
            if (vec && i + 4 <= it.size) {
                float4 p = *reinterpret_cast<const float4*>(it.values + i);
                const float4 g = *reinterpret_cast<const float4*>(it.grad + i);
                float4 m = *reinterpret_cast<const float4*>(it.m + i);
                float4 v = *reinterpret_cast<const float4*>(it.v + i);
                adamw_element(p.x, g.x, m.x, v.x, lr, b1, b2, it.c1, it.c2, eps, decay);
                adamw_element(p.y, g.y, m.y, v.y, lr, b1, b2, it.c1, it.c2, eps, decay);
                adamw_element(p.z, g.z, m.z, v.z, lr, b1, b2, it.c1, it.c2, eps, decay);
                adamw_element(p.w, g.w, m.w, v.w, lr, b1, b2, it.c1, it.c2, eps, decay);
                *reinterpret_cast<float4*>(it.values + i) = p;
                *reinterpret_cast<float4*>(it.m + i) = m;
                *reinterpret_cast<float4*>(it.v + i) = v;
                if (it.shadow) {
                    __nv_bfloat162 lo = __floats2bfloat162_rn(p.x, p.y), hi = __floats2bfloat162_rn(p.z, p.w);
                    uint2 packed;
                    packed.x = *reinterpret_cast<uint32_t*>(&lo);
                    packed.y = *reinterpret_cast<uint32_t*>(&hi);
                    *reinterpret_cast<uint2*>(it.shadow + i) = packed;
                }
            } else {
                for (long long j = i; j < i + 4 && j < it.size; ++j) {
                    float p = it.values[j], m = it.m[j], v = it.v[j];
                    adamw_element(p, it.grad[j], m, v, lr, b1, b2, it.c1, it.c2, eps, decay);
                    it.values[j] = p; it.m[j] = m; it.v[j] = v;
                    if (it.shadow) it.shadow[j] = __float2bfloat16_rn(p);
                }
            }
        }
    }
}

// Sum of squares of every gradient, in double, in a fixed order: block b takes chunks b, b + B, ...; its
// threads add their elements in index order and the block combines them with a fixed tree.
constexpr int kNormBlocks = 1024;
__global__ void __launch_bounds__(kOptimThreads)
grad_square_sum_kernel(const Item* __restrict__ items, int count, long long total_chunks, double* __restrict__ partial) {
    __shared__ double s_sum[kOptimThreads];
    double sum = 0.0;
    for (long long chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
        const Item it = items[find_item(items, count, chunk)];
        const long long base = (chunk - it.first_chunk) * kChunk;
        const bool vec = ((uintptr_t)it.grad & 15u) == 0;
#pragma unroll
        for (int r = 0; r < kChunk / (kOptimThreads * 4); ++r) {
            const long long i = base + ((long long)r * kOptimThreads + threadIdx.x) * 4;
            if (i >= it.size) break;
            if (vec && i + 4 <= it.size) {
                const float4 g = *reinterpret_cast<const float4*>(it.grad + i);
                sum += (double)g.x * g.x + (double)g.y * g.y + (double)g.z * g.z + (double)g.w * g.w;
            } else {
                for (long long j = i; j < i + 4 && j < it.size; ++j) sum += (double)it.grad[j] * it.grad[j];
            }
        }
    }
    s_sum[threadIdx.x] = sum;
    __syncthreads();
    for (int step = kOptimThreads / 2; step > 0; step >>= 1) {
        if (threadIdx.x < step) s_sum[threadIdx.x] += s_sum[threadIdx.x + step];
        __syncthreads();
    }
    if (threadIdx.x == 0) partial[blockIdx.x] = s_sum[0];
}

// result[0] = norm, result[1] = factor the gradients are scaled by (1 when the norm is within the limit,
// upstream: `if norm > max_norm: scale = max_norm / norm`, src/qutai/nn/optimizers.py:27-30)
__global__ void __launch_bounds__(kNormBlocks)
grad_norm_finish_kernel(const double* __restrict__ partial, int blocks, double max_norm, double* __restrict__ result) {
    __shared__ double s_sum[kNormBlocks];
    s_sum[threadIdx.x] = (int)threadIdx.x < blocks ? partial[threadIdx.x] : 0.0;
    __syncthreads();
    for (int step = kNormBlocks / 2; step > 0; step >>= 1) {
        if ((int)threadIdx.x < step) s_sum[threadIdx.x] += s_sum[threadIdx.x + step];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        const double norm = sqrt(s_sum[0]);
        result[0] = norm;
        result[1] = norm > max_norm ? max_norm / norm : 1.0;   // a NaN norm compares false: nothing is scaled
    }
}

__global__ void __launch_bounds__(kOptimThreads)
grad_scale_kernel(const Item* __restrict__ items, int count, long long total_chunks, const double* __restrict__ result) {
    const double factor = result[1];
    if (factor == 1.0) return;
    const float f = (float)factor;
    for (long long chunk = blockIdx.x; chunk < total_chunks; chunk += gridDim.x) {
        const Item it = items[find_item(items, count, chunk)];
        const long long base = (chunk - it.first_chunk) * kChunk;
        const bool vec = ((uintptr_t)it.grad & 15u) == 0;
#pragma unroll
        for (int r = 0; r < kChunk / (kOptimThreads * 4); ++r) {
            const long long i = base + ((long long)r * kOptimThreads + threadIdx.x) * 4;
            if (i >= it.size) break;
            if (vec && i + 4 <= it.size) {
                float4 g = *reinterpret_cast<const float4*>(it.grad + i);
                g.x *= f; g.y *= f; g.z *= f; g.w *= f;
                *reinterpret_cast<float4*>(it.grad + i) = g;
            } else {
                for (long long j = i; j < i + 4 && j < it.size; ++j) it.grad[j] *= f;
            }
        }
    }
}

// Validates the host table, fills in first_chunk, copies it to `table` on the device.  Returns the chunk total.
int stage_table(qmoe_optim_item_t* items, int count, uint64_t table, bool need_state, long long* total, cudaStream_t stream) {
    if (!items || count <= 0) return fail_arg("optimizer: the item table is empty");
    if (!table || (table & 15u)) return fail_arg("optimizer: the device table address must be non-null and 16-byte aligned");
    long long chunks = 0;
    for (int i = 0; i < count; ++i) {
        qmoe_optim_item_t& it = items[i];
        if (it.size <= 0) return fail_arg("optimizer: item %d has size %lld", i, (long long)it.size);
        if (!it.grad || (need_state && (!it.values || !it.exp_avg || !it.exp_avg_sq)))
            return fail_arg("optimizer: item %d has a null address", i);
        if ((it.grad | it.values | it.exp_avg | it.exp_avg_sq) & 3u || it.shadow & 1u)
            return fail_arg("optimizer: item %d has a misaligned address", i);
        it.first_chunk = chunks;
        chunks += (it.size + kChunk - 1) / kChunk;
    }
    *total = chunks;
    QMOE_CUDA(cudaMemcpyAsync((void*)table, items, (size_t)count * sizeof(qmoe_optim_item_t), cudaMemcpyHostToDevice, stream));
    return 0;
}

int stream_grid(long long chunks) {
    const long long cap = (long long)sm_count() * 8;
    return (int)(chunks < cap ? chunks : cap);
}

}  // namespace
}  // namespace qmoe

using namespace qmoe;

extern "C" int64_t qmoe_optim_table_bytes(int32_t count) { return (int64_t)(count > 0 ? count : 0) * (int64_t)sizeof(qmoe_optim_item_t); }

extern "C" int64_t qmoe_clip_scratch_bytes(void) { return (int64_t)(kNormBlocks + 2) * (int64_t)sizeof(double); }

extern "C" int qmoe_adamw_multi(qmoe_optim_item_t* items, int32_t count, uint64_t table, float learning_rate, float beta1,
                                float beta2, float eps, float weight_decay, uint64_t stream_) {
    if (learning_rate < 0 || eps < 0 || weight_decay < 0) return fail_arg("adamw: learning rate, eps and weight decay must not be negative");
    if (!(beta1 >= 0 && beta1 < 1 && beta2 >= 0 && beta2 < 1)) return fail_arg("adamw: betas must lie in [0, 1)");
    cudaStream_t stream = (cudaStream_t)stream_;
    for (int i = 0; items && i < count; ++i)
        if (!(items[i].c1 > 0) || !(items[i].c2 > 0)) return fail_arg("adamw: item %d has a non-positive bias correction", i);
    long long chunks = 0;
    if (int rc = stage_table(items, count, table, true, &chunks, stream)) return rc;
    TimedScope timed(KC_OPTIMIZER, stream);
    adamw_multi_kernel<<<stream_grid(chunks), kOptimThreads, 0, stream>>>((const Item*)table, count, chunks, learning_rate,
                                                                         beta1, beta2, eps, weight_decay);
    QMOE_LAUNCH_CHECK("adamw_multi_kernel");
    return 0;
}

extern "C" int qmoe_clip_grad_norm(qmoe_optim_item_t* items, int32_t count, uint64_t table, double max_norm,
                                   uint64_t scratch, uint64_t stream_) {
    if (!(max_norm >= 0) || max_norm > 1.7e308) return fail_arg("clip_grad_norm: max_norm must be a non-negative finite number");
    if (!scratch || (scratch & 7u)) return fail_arg("clip_grad_norm: scratch must be non-null and 8-byte aligned");
    cudaStream_t stream = (cudaStream_t)stream_;
    long long chunks = 0;
    if (int rc = stage_table(items, count, table, false, &chunks, stream)) return rc;
    TimedScope timed(KC_OPTIMIZER, stream);
    double* result = (double*)scratch;       // [0] norm, [1] factor
    double* partial = result + 2;            // [kNormBlocks]
    const int blocks = (int)(chunks < kNormBlocks ? chunks : kNormBlocks);
    grad_square_sum_kernel<<<blocks, kOptimThreads, 0, stream>>>((const Item*)table, count, chunks, partial);
    QMOE_LAUNCH_CHECK("grad_square_sum_kernel");
    grad_norm_finish_kernel<<<1, kNormBlocks, 0, stream>>>(partial, blocks, max_norm, result);
    QMOE_LAUNCH_CHECK("grad_norm_finish_kernel");
    grad_scale_kernel<<<stream_grid(chunks), kOptimThreads, 0, stream>>>((const Item*)table, count, chunks, result);
    QMOE_LAUNCH_CHECK("grad_scale_kernel");
    return 0;
}
