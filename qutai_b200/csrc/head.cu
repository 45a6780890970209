// The language-model head with its cross-entropy loss: loss = mean over counted rows of
//     log sum_c exp(logits[r, c]) - logits[r, label(r)],   logits = hidden_rows . weight^T
// (upstream: projection_loss src/qutai/lm/layers.py:187-257; kernels lm_head_rows, lm_head_loss, lm_head_gradient
// src/qutai/backends/cuda/lm.cu:430-444; CPU statement src/qutai/backends/cpu_lm.py:323-371).  Upstream walks the rows in
// chunks so that the [rows, vocab] logits never exist as a whole, and therefore forms every chunk's logits twice (once
// for the loss, once more in the backward) and reads them four times.  With 180 GB of HBM the logits of a whole step
// fit (8188 rows x 32000 classes in bf16 = 0.5 GB), so here
//   * the rows that have a target (every position but the last of each sequence) are gathered once;
//   * ONE product forms the logits (grouped tcgen05 kernel with a single group; CUDA cores for fp32);
//   * ONE pass over the logits leaves each row's loss and overwrites the row with its gradient
//     (softmax - one_hot) / count: a row is read from HBM once, kept in shared memory, written once;
//   * the backward is the two remaining products (input gradient, weight gradient) on the kept gradient, scaled by
//     the incoming scalar afterwards when there is one.
// Sums over rows run in a fixed order (no floating-point atomics).
#include "common.cuh"

namespace qmoe {
namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr long long kMaxCachedRowBytes = 200 * 1024;   // a row of logits kept in shared memory while it is worked on

// exp and log in the precision the row is stored in: bf16 rows take the fast forms (their results are rounded to 8 bits
// of mantissa anyway), fp32 rows, the parity mode, the accurate ones
template <typename T> __device__ __forceinline__ float exp_for(float v) { return sizeof(T) == 2 ? __expf(v) : expf(v); }
template <typename T> __device__ __forceinline__ float log_for(float v) { return sizeof(T) == 2 ? __logf(v) : logf(v); }

__device__ __forceinline__ float block_max(float v, float* tmp) {
    v = warp_max(v);
    __syncthreads();   // tmp may still be read from the reduction before
    if ((threadIdx.x & 31) == 0) tmp[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = tmp[0];
#pragma unroll
    for (int i = 1; i < kWarps; ++i) r = fmaxf(r, tmp[i]);
    return r;
}
__device__ __forceinline__ float block_sum(float v, float* tmp) {
    v = warp_sum(v);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) tmp[threadIdx.x >> 5] = v;
    __syncthreads();
    float r = tmp[0];
#pragma unroll
    for (int i = 1; i < kWarps; ++i) r += tmp[i];   // the same order in every thread and every run
    return r;
}

// Label of head row r: the token that follows position (r mod (time - 1)) of sequence r / (time - 1).  A value
// outside [0, vocab) is returned as -100 (not counted), so that no label can send a read outside its row.
// time == 0: `labels` is the flat list of targets (one per head row), as upstream's prepared labels are.
__device__ __forceinline__ long long label_of(const long long* labels, long long r, int time, long long vocab) {
    const long long label = time ? labels[(r / (time - 1)) * time + r % (time - 1) + 1] : labels[r];
    return label >= 0 && label < vocab ? label : -100;
}

// meta[0] = number of rows with a label other than -100 (at least 1, as upstream divides), as a float: 1 / that
__global__ void __launch_bounds__(1024) head_count_kernel(const long long* __restrict__ labels, long long rows, int time,
                                                          long long vocab, float* __restrict__ factor, int* __restrict__ group,
                                                          int rows_bound) {
    __shared__ int tmp[32];
    int mine = 0;
    for (long long r = threadIdx.x; r < rows; r += blockDim.x) mine += label_of(labels, r, time, vocab) != -100;
#pragma unroll
    for (int o = 16; o; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if ((threadIdx.x & 31) == 0) tmp[threadIdx.x >> 5] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        int total = 0;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += tmp[i];
        factor[0] = 1.f / (float)(total > 1 ? total : 1);
        // the one group of the grouped products: offsets {0, rows_bound}, counts {rows}
        group[0] = 0; group[1] = rows_bound; group[2] = (int)rows; group[3] = 0;
    }
}

// inputs[r, :] = hidden[(r / (time - 1)) * time + r % (time - 1), :] for r < rows, zero for the pad rows up to rows_bound
// (backward == 0); d_hidden[b, t, :] = d_inputs[b * (time - 1) + t, :] for t < time - 1, zero for the last position
// (backward != 0).  16-byte pieces.
__global__ void __launch_bounds__(256) head_rows_kernel(const uint4* __restrict__ src, uint4* __restrict__ dst, long long dst_rows,
                                                        long long rows, int time, long long pieces, int backward) {
    const long long total = dst_rows * pieces;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long row = i / pieces, piece = i - row * pieces;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (!backward) {
            if (row < rows) v = src[((row / (time - 1)) * time + row % (time - 1)) * pieces + piece];
        } else {
            const long long t = row % time;
            if (t < time - 1) v = src[((row / time) * (time - 1) + t) * pieces + piece];
        }
        dst[i] = v;
    }
}

// One block per row: row_loss[r] (when given) and, in place (when write_gradient), factor[0] * (softmax - one_hot).
// CACHED: the row is read from global memory once and kept in shared memory (in its storage type).
template <typename T, bool CACHED>
__global__ void __launch_bounds__(kThreads)
head_loss_gradient_kernel(T* __restrict__ logits, const long long* __restrict__ labels, const float* __restrict__ factor,
                          float* __restrict__ row_loss, long long rows, long long vocab, int time, int write_gradient) {
    extern __shared__ __align__(16) uint8_t cache_raw[];
    __shared__ float tmp[kWarps];
    T* cache = reinterpret_cast<T*>(cache_raw);
    constexpr int N = Vec16<T>::N;
    const long long r = blockIdx.x;
    if (r >= rows) return;
    T* row = logits + r * vocab;
    const long long label = label_of(labels, r, time, vocab);
    const bool vec = vocab % N == 0 && (reinterpret_cast<uintptr_t>(row) & 15u) == 0;
    const int pieces = vec ? (int)(vocab / N) : 0;
    if (label == -100) {   // not counted: no loss, no gradient
        if (write_gradient) {
            if (vec) for (int c = threadIdx.x; c < pieces; c += kThreads) reinterpret_cast<uint4*>(row)[c] = make_uint4(0, 0, 0, 0);
            else for (long long c = threadIdx.x; c < vocab; c += kThreads) Act<T>::store(row + c, 0.f);
        }
        if (threadIdx.x == 0 && row_loss) row_loss[r] = 0.f;
        return;
    }
    const T* from = CACHED ? cache : row;
    float peak = -INFINITY;
    if (vec) {
        for (int c = threadIdx.x; c < pieces; c += kThreads) {
            const uint4 v = reinterpret_cast<const uint4*>(row)[c];
            if (CACHED) reinterpret_cast<uint4*>(cache)[c] = v;
            float f[N];
            Vec16<T>::unpack(v, f);
#pragma unroll
            for (int i = 0; i < N; ++i) peak = fmaxf(peak, f[i]);
        }
    } else {
        for (long long c = threadIdx.x; c < vocab; c += kThreads) {
            const float v = Act<T>::load(row + c);
            if (CACHED) cache[c] = row[c];
            peak = fmaxf(peak, v);
        }
    }
    peak = block_max(peak, tmp);   // its barriers also publish the cache
    float total = 0.f;
    if (vec) {
        for (int c = threadIdx.x; c < pieces; c += kThreads) {
            float f[N];
            Vec16<T>::unpack(reinterpret_cast<const uint4*>(from)[c], f);
#pragma unroll
            for (int i = 0; i < N; ++i) total += exp_for<T>(f[i] - peak);
        }
    } else {
        for (long long c = threadIdx.x; c < vocab; c += kThreads) total += exp_for<T>(Act<T>::load(from + c) - peak);
    }
    total = block_sum(total, tmp);
    if (threadIdx.x == 0 && row_loss) row_loss[r] = log_for<T>(total) - (Act<T>::load(from + label) - peak);
    if (!write_gradient) return;
    __syncthreads();   // the label's logit has been read before anything is overwritten (uncached form)
    const float scale = factor[0], inverse = 1.f / total;
    if (vec) {
        for (int c = threadIdx.x; c < pieces; c += kThreads) {
            float f[N];
            Vec16<T>::unpack(reinterpret_cast<const uint4*>(from)[c], f);
#pragma unroll
            for (int i = 0; i < N; ++i) f[i] = scale * (exp_for<T>(f[i] - peak) * inverse - ((long long)c * N + i == label ? 1.f : 0.f));
            reinterpret_cast<uint4*>(row)[c] = Vec16<T>::pack(f);
        }
    } else {
        for (long long c = threadIdx.x; c < vocab; c += kThreads)
            Act<T>::store(row + c, scale * (exp_for<T>(Act<T>::load(from + c) - peak) * inverse - (c == label ? 1.f : 0.f)));
    }
}

// loss[0] = factor * sum_r row_loss[r], one block, fixed order
__global__ void __launch_bounds__(1024) head_mean_kernel(const float* __restrict__ row_loss, const float* __restrict__ factor,
                                                         float* __restrict__ loss, long long rows) {
    __shared__ float tmp[32];
    float mine = 0.f;
    for (long long r = threadIdx.x; r < rows; r += blockDim.x) mine += row_loss[r];
    mine = warp_sum(mine);
    if ((threadIdx.x & 31) == 0) tmp[threadIdx.x >> 5] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += tmp[i];
        loss[0] = total * factor[0];
    }
}

// values[i] *= scalar[0]
template <typename T>
__global__ void __launch_bounds__(256) head_scale_kernel(T* __restrict__ values, const float* __restrict__ scalar, long long n) {
    const float s = scalar[0];
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        Act<T>::store(values + i, Act<T>::load(values + i) * s);
}

int check_head(const qmoe_head_t* h) {
    if (!h) return fail_arg("head is null");
    if (h->dtype != QMOE_BF16 && h->dtype != QMOE_F32) return fail_arg("head: dtype must be QMOE_F32 or QMOE_BF16");
    if (h->batch <= 0 || h->time < 2 || h->width <= 0 || h->vocab <= 0) return fail_arg("head: batch, width, vocab must be positive and time at least 2");
    const long long rows = (long long)h->batch * (h->time - 1);
    if (h->rows_bound < rows || h->rows_bound % kRowPad) return fail_arg("head: rows_bound must cover batch * (time - 1) rows and be a multiple of %d", kRowPad);
    if (h->rows_bound > 0x7fffffffll) return fail_arg("head: too many rows");
    const long long element = h->dtype == QMOE_BF16 ? 2 : 4;
    if ((h->width * element) % 16) return fail_arg("head: a row of hidden must be a multiple of 16 bytes");
    if (!h->hidden || !h->weight || !h->labels || !h->inputs || !h->logits || !h->row_loss || !h->loss || !h->meta)
        return fail_arg("head: null buffer address");
    if ((h->hidden | h->inputs | h->logits) & 15u) return fail_arg("head: buffers must be 16-byte aligned");
    return 0;
}
bool head_on_tensor_cores(const qmoe_head_t* h) { return h->dtype == QMOE_BF16 && tcgen05_shape_ok(h->width, h->vocab); }
qmoe_route_t one_group(const qmoe_head_t* h) {   // the fields the grouped tensor-core products read
    qmoe_route_t r = {};
    r.rows_bound = h->rows_bound;
    r.offsets = h->meta + 16;   // i32 {0, rows_bound}
    r.counts = h->meta + 24;    // i32 {rows}
    return r;
}
int grid_for(long long n) { const long long blocks = (n + 255) / 256; return (int)(blocks > 8 * 148 ? 8 * 148 : blocks); }

// the loss pass over `rows` rows of logits: row losses (row_loss may be null) and / or the gradient in place
template <typename T>
int launch_loss_pass(T* logits, const long long* labels, const float* factor, float* row_loss, long long rows, long long vocab,
                     int time, int write_gradient, cudaStream_t stream) {
    const long long bytes = vocab * (long long)sizeof(T);
    if (bytes <= kMaxCachedRowBytes) {
        auto kernel = head_loss_gradient_kernel<T, true>;
        const int smem = (int)((bytes + 15) / 16 * 16);
        QMOE_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxCachedRowBytes));
        kernel<<<(unsigned)rows, kThreads, smem, stream>>>(logits, labels, factor, row_loss, rows, vocab, time, write_gradient);
    } else {
        head_loss_gradient_kernel<T, false><<<(unsigned)rows, kThreads, 0, stream>>>(logits, labels, factor, row_loss, rows, vocab, time,
                                                                                      write_gradient);
    }
    QMOE_LAUNCH_CHECK("head_loss_gradient_kernel");
    return 0;
}
template <typename T>
int launch_loss_gradient(const qmoe_head_t* h, long long rows, cudaStream_t stream) {
    return launch_loss_pass<T>((T*)h->logits, (const long long*)h->labels, (const float*)h->meta, (float*)h->row_loss, rows, h->vocab,
                               h->time, 1, stream);
}

// rows [start, start + count) of the head's inputs: out[i, :] = values[position(start + i), :] (backward == 0) or
// target[position(start + i), :] += gradient[i, :] (backward != 0); position(r) = (r / (time - 1)) * time + r % (time - 1)
template <typename T>
__global__ void __launch_bounds__(256) head_rows_range_kernel(const T* __restrict__ src, T* __restrict__ dst, long long start,
                                                              long long count, long long width, int time, int backward) {
    const long long total = count * width;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const long long row = start + i / width, at = ((row / (time - 1)) * time + row % (time - 1)) * width + i % width;
        if (backward) Act<T>::store(dst + at, Act<T>::load(dst + at) + Act<T>::load(src + i));
        else dst[i] = src[at];
    }
}
// out[0] = scale * sum of values (fixed order); scale = numerator[0] / denominator when numerator is given
__global__ void __launch_bounds__(1024) head_sum_kernel(const float* __restrict__ values, float* __restrict__ out, long long n) {
    __shared__ float tmp[32];
    float mine = 0.f;
    for (long long r = threadIdx.x; r < n; r += blockDim.x) mine += values[r];
    mine = warp_sum(mine);
    if ((threadIdx.x & 31) == 0) tmp[threadIdx.x >> 5] = mine;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.f;
        for (int i = 0; i < (int)(blockDim.x >> 5); ++i) total += tmp[i];
        out[0] = total;
    }
}
__global__ void head_factor_kernel(const float* __restrict__ gradient, float count, float* __restrict__ factor) {
    factor[0] = gradient[0] / count;
}

}  // namespace
}  // namespace qmoe

using namespace qmoe;

extern "C" int qmoe_head_forward(const qmoe_head_t* h, uint64_t stream_) {
    if (int rc = check_head(h)) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    const long long rows = (long long)h->batch * (h->time - 1), element = h->dtype == QMOE_BF16 ? 2 : 4;
    {
        TimedScope timed(KC_OTHER, stream);
        head_count_kernel<<<1, 1024, 0, stream>>>((const long long*)h->labels, rows, h->time, h->vocab, (float*)h->meta, (int*)(h->meta + 16),
                                                  (int)h->rows_bound);
        QMOE_LAUNCH_CHECK("head_count_kernel");
        const long long pieces = h->width * element / 16;
        head_rows_kernel<<<grid_for(h->rows_bound * pieces), 256, 0, stream>>>((const uint4*)h->hidden, (uint4*)h->inputs, h->rows_bound, rows,
                                                                               h->time, pieces, 0);
        QMOE_LAUNCH_CHECK("head_rows_kernel");
    }
    {
        TimedScope timed(KC_EXPERT_GEMM, stream);
        if (head_on_tensor_cores(h)) {
            const qmoe_route_t r = one_group(h);
            if (int rc = tc_rows_nt(&r, 1, h->inputs, h->weight, h->logits, h->width, h->vocab, stream, nullptr)) return rc;
        } else {
            SimtGemmArgs g = {};
            g.A = (const void*)h->inputs; g.B = (const void*)h->weight; g.C = (void*)h->logits;
            g.M = rows; g.N = h->vocab; g.K = h->width;
            g.a_rs = h->width; g.a_cs = 1; g.b_rs = 1; g.b_cs = h->width;
            g.ldc = h->vocab; g.mode = SG_PLAIN;
            if (int rc = launch_simt_gemm(g, h->dtype, h->dtype, h->dtype, rows, 1, stream)) return rc;
        }
    }
    TimedScope timed(KC_HEAD_LOSS, stream);
    if (int rc = h->dtype == QMOE_BF16 ? launch_loss_gradient<__nv_bfloat16>(h, rows, stream) : launch_loss_gradient<float>(h, rows, stream)) return rc;
    head_mean_kernel<<<1, 1024, 0, stream>>>((const float*)h->row_loss, (const float*)h->meta, (float*)h->loss, rows);
    QMOE_LAUNCH_CHECK("head_mean_kernel");
    return 0;
}

extern "C" int qmoe_head_backward(const qmoe_head_t* h, uint64_t gradient, uint64_t stream_) {
    if (int rc = check_head(h)) return rc;
    if (!h->d_hidden && !h->d_weight) return fail_arg("head_backward: nothing to compute");
    if (h->d_hidden && !h->d_inputs) return fail_arg("head_backward: d_inputs is needed for d_hidden");
    cudaStream_t stream = (cudaStream_t)stream_;
    const long long rows = (long long)h->batch * (h->time - 1), element = h->dtype == QMOE_BF16 ? 2 : 4;
    const bool tensor_cores = head_on_tensor_cores(h);
    const qmoe_route_t r = one_group(h);
    if (h->d_hidden) {
        {
            TimedScope timed(KC_EXPERT_GEMM, stream);
            if (tensor_cores) {
                if (int rc = tc_rows_nn(&r, 1, h->logits, h->weight, 0, 0, h->d_inputs, h->vocab, h->width, stream, nullptr)) return rc;
            } else {
                SimtGemmArgs g = {};
                g.A = (const void*)h->logits; g.B = (const void*)h->weight; g.C = (void*)h->d_inputs;
                g.M = rows; g.N = h->width; g.K = h->vocab;
                g.a_rs = h->vocab; g.a_cs = 1; g.b_rs = h->width; g.b_cs = 1;
                g.ldc = h->width; g.mode = SG_PLAIN;
                if (int rc = launch_simt_gemm(g, h->dtype, h->dtype, h->dtype, rows, 1, stream)) return rc;
            }
        }
        TimedScope timed(KC_OTHER, stream);
        const long long pieces = h->width * element / 16, hidden_rows = (long long)h->batch * h->time;
        head_rows_kernel<<<grid_for(hidden_rows * pieces), 256, 0, stream>>>((const uint4*)h->d_inputs, (uint4*)h->d_hidden, hidden_rows, rows,
                                                                             h->time, pieces, 1);
        QMOE_LAUNCH_CHECK("head_rows_kernel");
        if (gradient) {
            if (h->dtype == QMOE_BF16) head_scale_kernel<<<grid_for(hidden_rows * h->width), 256, 0, stream>>>((__nv_bfloat16*)h->d_hidden, (const float*)gradient, hidden_rows * h->width);
            else head_scale_kernel<<<grid_for(hidden_rows * h->width), 256, 0, stream>>>((float*)h->d_hidden, (const float*)gradient, hidden_rows * h->width);
            QMOE_LAUNCH_CHECK("head_scale_kernel");
        }
    }
    if (h->d_weight) {
        {
            TimedScope timed(KC_WGRAD_GEMM, stream);
            if (tensor_cores) {
                if (int rc = tc_wgrad1(&r, h->logits, h->inputs, h->d_weight, h->vocab, h->width, stream)) return rc;
            } else {
                SimtGemmArgs g = {};
                g.A = (const void*)h->logits; g.B = (const void*)h->inputs; g.C = (void*)h->d_weight;
                g.M = h->vocab; g.N = h->width; g.K = rows;
                g.a_rs = 1; g.a_cs = h->vocab; g.b_rs = h->width; g.b_cs = 1;
                g.ldc = h->width; g.mode = SG_PLAIN;
                if (int rc = launch_simt_gemm(g, h->dtype, h->dtype, QMOE_F32, h->vocab, 1, stream)) return rc;
            }
        }
        if (gradient) {
            TimedScope timed(KC_OTHER, stream);
            head_scale_kernel<<<grid_for(h->vocab * h->width), 256, 0, stream>>>((float*)h->d_weight, (const float*)gradient, h->vocab * h->width);
            QMOE_LAUNCH_CHECK("head_scale_kernel");
        }
    }
    return 0;
}

// ---- the per-chunk functions of upstream's backend table (src/qutai/backends/cuda_lm.py:584-660) -----------------
extern "C" int qmoe_head_rows(uint64_t values, uint64_t out, int32_t dtype, int64_t start, int64_t count, int64_t width,
                              int64_t time, int32_t backward, uint64_t stream_) {
    if (!values || !out) return fail_arg("head_rows: null address");
    if (start < 0 || count <= 0 || width <= 0 || time < 2) return fail_arg("head_rows: sizes must be positive and time at least 2");
    if (dtype != QMOE_BF16 && dtype != QMOE_F32) return fail_arg("head_rows: dtype must be QMOE_F32 or QMOE_BF16");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_OTHER, stream);
    // forward: values = hidden, out = the rows; backward: values = the rows' gradient, out = the hidden gradient added to
    if (dtype == QMOE_BF16)
        head_rows_range_kernel<<<grid_for(count * width), 256, 0, stream>>>((const __nv_bfloat16*)values, (__nv_bfloat16*)out, start, count, width,
                                                                            (int)time, backward);
    else
        head_rows_range_kernel<<<grid_for(count * width), 256, 0, stream>>>((const float*)values, (float*)out, start, count, width, (int)time,
                                                                            backward);
    QMOE_LAUNCH_CHECK("head_rows_range_kernel");
    return 0;
}

extern "C" int qmoe_head_loss(uint64_t logits, int32_t dtype, uint64_t labels, uint64_t row_loss, uint64_t out, int64_t rows,
                              int64_t vocab, int64_t start, uint64_t stream_) {
    if (!logits || !labels || !row_loss || !out) return fail_arg("head_loss: null address");
    if (rows <= 0 || vocab <= 0 || start < 0) return fail_arg("head_loss: sizes must be positive");
    if (dtype != QMOE_BF16 && dtype != QMOE_F32) return fail_arg("head_loss: dtype must be QMOE_F32 or QMOE_BF16");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_OTHER, stream);
    const long long* targets = (const long long*)labels + start;
    if (int rc = dtype == QMOE_BF16 ? launch_loss_pass<__nv_bfloat16>((__nv_bfloat16*)logits, targets, nullptr, (float*)row_loss, rows, vocab, 0, 0, stream)
                                    : launch_loss_pass<float>((float*)logits, targets, nullptr, (float*)row_loss, rows, vocab, 0, 0, stream))
        return rc;
    head_sum_kernel<<<1, 1024, 0, stream>>>((const float*)row_loss, (float*)out, rows);
    QMOE_LAUNCH_CHECK("head_sum_kernel");
    return 0;
}

extern "C" int qmoe_head_gradient(uint64_t logits, int32_t dtype, uint64_t labels, uint64_t gradient, uint64_t factor, int64_t count,
                                  int64_t rows, int64_t vocab, int64_t start, uint64_t stream_) {
    if (!logits || !labels || !gradient || !factor) return fail_arg("head_gradient: null address");
    if (rows <= 0 || vocab <= 0 || start < 0 || count <= 0) return fail_arg("head_gradient: sizes must be positive");
    if (dtype != QMOE_BF16 && dtype != QMOE_F32) return fail_arg("head_gradient: dtype must be QMOE_F32 or QMOE_BF16");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_OTHER, stream);
    head_factor_kernel<<<1, 1, 0, stream>>>((const float*)gradient, (float)count, (float*)factor);
    QMOE_LAUNCH_CHECK("head_factor_kernel");
    const long long* targets = (const long long*)labels + start;
    return dtype == QMOE_BF16 ? launch_loss_pass<__nv_bfloat16>((__nv_bfloat16*)logits, targets, (const float*)factor, nullptr, rows, vocab, 0, 1, stream)
                              : launch_loss_pass<float>((float*)logits, targets, (const float*)factor, nullptr, rows, vocab, 0, 1, stream);
}
