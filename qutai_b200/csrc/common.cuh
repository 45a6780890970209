// Shared declarations for libqutai_moe.so (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/qutai_moe.h"

namespace qmoe {

// Rows of every expert group in the permuted ("dispatched") layout are padded to a multiple of
// this, so that a 128-row tensor-core tile never straddles two experts.  Pad rows hold zeros.
constexpr int kRowPad = QMOE_ROW_PAD;
constexpr int kMaxExperts = QMOE_MAX_EXPERTS;
constexpr int kMaxTopK = QMOE_MAX_TOP_K;
// Token rows handled by one block of the routing kernels (8 warps x 4 rows): small blocks keep all SMs
// busy when a rank holds only a few thousand tokens.
constexpr int kRouteRowsPerBlock = 32;

// ---- error plumbing -------------------------------------------------------------------------
void set_error(const char* fmt, ...);
int fail_arg(const char* fmt, ...);                       // returns QMOE_ERR_ARGUMENT
int check_cuda(cudaError_t code, const char* what);       // 0 or positive cudaError_t
#define QMOE_CUDA(expr)                                  \
    do {                                                 \
        int _rc = ::qmoe::check_cuda((expr), #expr);     \
        if (_rc) return _rc;                             \
    } while (0)
#define QMOE_LAUNCH_CHECK(name)                          \
    do {                                                 \
        int _rc = ::qmoe::after_launch(name);            \
        if (_rc) return _rc;                             \
    } while (0)
int after_launch(const char* name);  // cudaGetLastError (+ sync when QUTAI_MOE_SYNC=1) + counters

// per-kernel-class timing (off unless enabled through the ABI)
enum KernelClass {
    KC_ROUTER_GEMM = 0, KC_ROUTE, KC_PERMUTE, KC_EXPERT_GEMM, KC_SWIGLU, KC_COMBINE, KC_COMBINE_BWD,
    KC_WGRAD_GEMM, KC_UNPERMUTE, KC_ROUTE_BWD, KC_CAST, KC_OTHER, KC_EXCHANGE, KC_OPTIMIZER, KC_NORM, KC_ATTENTION,
    KC_HEAD_LOSS, KC_ELEMENTWISE, KC_BARRIER, KC_ALL_REDUCE, KC_COUNT
};
struct TimedScope {  // records a pair of events around the launches made while it is alive
    TimedScope(KernelClass kc, cudaStream_t s);
    ~TimedScope();
    int slot;
    cudaStream_t stream;
};

// ---- small device helpers -------------------------------------------------------------------
template <typename T> struct Act;
template <> struct Act<float> {
    static __device__ __forceinline__ float load(const float* p) { return *p; }
    static __device__ __forceinline__ void store(float* p, float v) { *p = v; }
    static constexpr int kVec = 4;  // elements per 16-byte access
};
template <> struct Act<__nv_bfloat16> {
    static __device__ __forceinline__ float load(const __nv_bfloat16* p) { return __bfloat162float(*p); }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }
    static constexpr int kVec = 8;
};

// 16-byte vector of activations unpacked to floats and back
template <typename T> struct Vec16;
template <> struct Vec16<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
        f[0] = __uint_as_float(v.x); f[1] = __uint_as_float(v.y);
        f[2] = __uint_as_float(v.z); f[3] = __uint_as_float(v.w);
    }
    static __device__ __forceinline__ uint4 pack(const float* f) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]), __float_as_uint(f[3]));
    }
};
template <> struct Vec16<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void unpack(const uint4& v, float* f) {
        const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ uint4 pack(const float* f) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

__device__ __forceinline__ float sigmoid_stable(float v) {
    // two-branch logistic: never exponentiates a positive number
    if (v >= 0.f) return 1.f / (1.f + __expf(-v));
    float e = __expf(v);
    return e / (1.f + e);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

inline int ceil_div(long long a, long long b) { return (int)((a + b - 1) / b); }
int sm_count();

// ---- CUDA-core GEMM descriptor (gemm_simt.cu) ------------------------------------------------
enum SimtGroupMode { SG_PLAIN = 0, SG_ROWS = 1, SG_K = 2, SG_SPLITK = 3 };
struct SimtGemmArgs {
    const void* A;
    const void* B;
    void* C;
    const void* A2;  // optional second segment (same shapes and strides), may be null
    const void* B2;
    long long M, N, K;
    long long a_rs, a_cs;  // A(m, k) = A[m * a_rs + k * a_cs]
    long long b_rs, b_cs;  // B(k, n) = B[k * b_rs + n * b_cs]
    long long ldc;         // C(m, n) = C[m * ldc + n]
    int accumulate;
    int mode;
    const int* tile_expert;  // SG_ROWS: expert of each kRowPad-row tile of the dispatched layout
    const int* offsets;      // SG_K: first dispatched row of each expert
    const int* counts;       // SG_K: rows of each expert
    const int* meta;         // SG_ROWS: meta[0] = dispatched rows in use
    long long b_slab;        // SG_ROWS: elements of B per expert
    long long c_slab;        // SG_K / SG_SPLITK: elements of C per expert / per split
    long long k_chunk;       // SG_SPLITK: K handled by one split
};
// dtype codes QMOE_F32 / QMOE_BF16 for A, B, C; m_extent = rows the grid must cover
int launch_simt_gemm(const SimtGemmArgs& g, int a_dtype, int b_dtype, int c_dtype, long long m_extent, int groups,
                     cudaStream_t stream);

// ---- cross-file entry points -----------------------------------------------------------------
int route_check(const qmoe_route_t* r);
int launch_swiglu(const qmoe_route_t* r, uint64_t g, uint64_t u, uint64_t h, int dtype, long long hidden, cudaStream_t stream);
int launch_swiglu_backward(const qmoe_route_t* r, uint64_t dh, uint64_t g, uint64_t u, uint64_t dg, uint64_t du, int dtype,
                           long long hidden, cudaStream_t stream);
bool tcgen05_shape_ok(long long width, long long hidden);
int tc_swiglu_forward(const qmoe_route_t* r, const qmoe_experts_t* ex, uint64_t x, uint64_t g, uint64_t u, uint64_t h, cudaStream_t stream);
// optional "store each output row at its return address on the rank that owns it" for the bf16 row products
struct TcScatter {
    const int* ret;                 // [rows] rank << 26 | row
    unsigned long long base[16];    // destination buffer of every rank
};
int tc_rows_nt(const qmoe_route_t* r, int experts, uint64_t a, uint64_t b, uint64_t c, long long K, long long N, cudaStream_t stream,
               const TcScatter* scatter = nullptr);
int tc_rows_nn(const qmoe_route_t* r, int experts, uint64_t a, uint64_t b, uint64_t a2, uint64_t b2, uint64_t c, long long K,
               long long N, cudaStream_t stream, const TcScatter* scatter = nullptr);
int tc_dswiglu(const qmoe_route_t* r, int experts, uint64_t dy, uint64_t w_down, uint64_t g, uint64_t u, uint64_t dg,
               uint64_t du, long long d, long long h, cudaStream_t stream);
int tc_wgrad3(const qmoe_route_t* r, int experts, uint64_t dy, uint64_t h_act, uint64_t x, uint64_t dg, uint64_t du,
              uint64_t d_w_down, uint64_t d_w_gate, uint64_t d_w_up, long long d, long long h, cudaStream_t stream);
int tc_wgrad1(const qmoe_route_t* r, uint64_t a, uint64_t b, uint64_t out, long long M, long long N, cudaStream_t stream,
              int groups = 1, long long slab = 0);
int tc_router_forward(uint64_t x, uint64_t w3, uint64_t scores, long long T, long long d, int E, int S, cudaStream_t stream);
int tc_plain_f32_nn(uint64_t a, uint64_t b, uint64_t c, long long T, long long K, long long N, cudaStream_t stream);
int tc_split_wgrad(uint64_t a, long long a_pitch, uint64_t b, uint64_t partial, const int* offsets, const int* counts,
                   int splits, long long T, long long M, long long N, cudaStream_t stream);
int simt_router_logits(uint64_t x, int32_t x_dtype, uint64_t w_router, uint64_t scores, int64_t tokens, int64_t width,
                       int32_t experts, cudaStream_t stream);
int simt_router_backward(uint64_t d_scores, uint64_t x, int32_t x_dtype, uint64_t w_router, uint64_t dx_router,
                         uint64_t d_w_router, uint64_t partials, int64_t tokens, int64_t width, int32_t experts,
                         cudaStream_t stream);
long long simt_router_partials(int64_t tokens, int32_t experts, int64_t width);
int launch_reduce_partials(const float* partials, float* out, long long n, int splits, cudaStream_t stream);
void count_tensor_core_launch();
int kernel_variant(int which);  // 0 = default form, 1 = the comparison form selected by qmoe_test_select_variant
int* device_status_address();

}  // namespace qmoe
