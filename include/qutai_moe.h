/*
 * libqutai_moe.so — C ABI of the B200 (sm_100a) Mixture-of-Experts layer.
 *
 * This is the boundary a host binds with ctypes (or any FFI).  It replaces, for the MoE layer of
 * qutai.lm, the NVRTC source strings that the upstream CUDA backend launches from
 * src/qutai/backends/cuda_lm.py through src/qutai/backends/cuda_runtime.py:299-328.  Every entry
 * point is `extern "C"`, takes plain integers, sizes and device addresses (uint64_t, as the
 * upstream `_p()` helper passes them, src/qutai/backends/cuda.py:61-70) and returns an int:
 *
 *      0            success
 *    < 0            argument / state error (QMOE_ERR_*); the host raises ValueError, as the
 *                   upstream dispatcher does before any launch (src/qutai/backends/cuda.py:307-334)
 *    > 0            a cudaError_t (or 1000 + ncclResult_t); the host raises RuntimeError, as
 *                   src/qutai/backends/cuda_runtime.py:165-177 does for CUresult
 *
 * qmoe_last_error() returns the message of the last failure on the calling thread.
 *
 * Ownership: the library never owns tensors.  Inputs, outputs and scratch are allocated by the
 * caller and passed as device addresses; the library keeps only process-wide internals (cached
 * TMA descriptors, timing events, an optional NCCL communicator).  All work is enqueued on the
 * stream argument (0 = the legacy default stream, which is what the upstream runtime uses,
 * src/qutai/backends/cuda_runtime.py:326) of the CURRENT device/context; nothing synchronises
 * unless documented.
 *
 * Layouts.  T tokens, E experts, k = top_k, A = T*k assignments, d = model width, h = expert
 * hidden width.  All matrices are dense row-major.  The "dispatched" layout holds the rows routed
 * to expert 0, then expert 1, ...; inside one expert rows keep increasing (token, slot) order —
 * the order of the upstream `ids`/`slots` lists (src/qutai/backends/cpu_lm.py:204-221,
 * src/qutai/backends/cuda/lm.cu:353-383) — and each expert group starts at a multiple of
 * QMOE_ROW_PAD rows; the pad rows hold zeros.  A buffer in that layout has
 * qmoe_rows_bound(T, E, k) rows.
 */
#ifndef QUTAI_MOE_H
#define QUTAI_MOE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define QMOE_VERSION 100
#define QMOE_ROW_PAD 128
#define QMOE_MAX_EXPERTS 256
#define QMOE_MAX_TOP_K 8

enum {
    QMOE_OK = 0,
    QMOE_ERR_ARGUMENT = -1,    /* bad size, null address, misaligned buffer */
    QMOE_ERR_UNSUPPORTED = -2, /* shape or dtype this build has no kernel for */
    QMOE_ERR_STATE = -3,       /* call order / initialisation problem */
    QMOE_ERR_DEVICE_CHECK = -4 /* a kernel recorded a failed self-check (bounded wait ran out, bad table) */
};

enum { QMOE_F32 = 0, QMOE_BF16 = 1 };                     /* activation dtype */
enum { QMOE_ENGINE_AUTO = 0, QMOE_ENGINE_SIMT = 1, QMOE_ENGINE_TCGEN05 = 2 };

/* ---------------------------------------------------------------------------------------------
 * Library, device memory and stream helpers.  They let a dependency-free host keep device
 * buffers, the role src/qutai/backends/cuda_runtime.py:184-258 (allocate/free/upload/download)
 * plays upstream.  A host that already owns device memory does not need them.
 * ------------------------------------------------------------------------------------------- */
int qmoe_version(void);
const char* qmoe_last_error(void);
int qmoe_device_info(int* sm_count, int* cc_major, int* cc_minor, uint64_t* total_bytes);
int qmoe_malloc(uint64_t* address, uint64_t bytes);
int qmoe_free(uint64_t address);
int qmoe_host_alloc(void** host, uint64_t bytes);         /* pinned host memory */
int qmoe_host_free(void* host);
int qmoe_memcpy_h2d(uint64_t dst, const void* src, uint64_t bytes, uint64_t stream);
int qmoe_memcpy_d2h(void* dst, uint64_t src, uint64_t bytes, uint64_t stream); /* async; sync the stream before reading */
int qmoe_memcpy_d2d(uint64_t dst, uint64_t src, uint64_t bytes, uint64_t stream);
int qmoe_memset(uint64_t dst, int value, uint64_t bytes, uint64_t stream);
int qmoe_stream_sync(uint64_t stream);
/* Extra streams and events (cudaStreamNonBlocking / timing disabled) for hosts that overlap copies or
 * exchanges with compute; the upstream runtime has a single stream (src/qutai/backends/cuda_runtime.py:326). */
int qmoe_stream_create(uint64_t* stream);
int qmoe_stream_destroy(uint64_t stream);
int qmoe_event_create(uint64_t* event);
int qmoe_event_destroy(uint64_t event);
int qmoe_event_record(uint64_t event, uint64_t stream);
int qmoe_stream_wait_event(uint64_t stream, uint64_t event);
int qmoe_event_sync(uint64_t event);                       /* host waits for the event only */
/* CUDA graphs (no upstream counterpart: its runtime launches kernel by kernel,
 * src/qutai/backends/cuda_runtime.py:299-328).  Between qmoe_graph_begin and qmoe_graph_end every call of this
 * library on `stream` (a stream from qmoe_stream_create, not 0) is recorded instead of run; qmoe_graph_launch
 * replays the recording with the same addresses.  Run the same calls once without capture first (the first call
 * of a kernel configures it).  After an error inside a capture call qmoe_graph_abandon. */
int qmoe_graph_begin(uint64_t stream);
int qmoe_graph_end(uint64_t stream, uint64_t* graph);
int qmoe_graph_abandon(uint64_t stream);
int qmoe_graph_launch(uint64_t graph, uint64_t stream);
int qmoe_graph_destroy(uint64_t graph);
/* launches made by this library since load (the upstream runtime keeps the same counter,
 * src/qutai/backends/cuda_runtime.py:95, :327); tensor-core launches counted separately (:100). */
int64_t qmoe_launch_count(void);
int64_t qmoe_tensor_core_launch_count(void);
/* Per-kernel-class device timing with CUDA events on the launching stream.  enable=1 starts a
 * fresh measurement; qmoe_timing_read synchronises the device and returns, per class, the summed
 * milliseconds and the number of timed scopes.  Class names via qmoe_timing_class_name. */
int qmoe_timing_enable(int enable);
int qmoe_timing_classes(void);
const char* qmoe_timing_class_name(int kernel_class);
int qmoe_timing_read(double* milliseconds, int64_t* scopes, int capacity);
/* status word written by kernels that check themselves; 0 = clean.  Synchronises the stream. */
int qmoe_device_status(uint64_t stream, int* status);
int qmoe_device_status_clear(uint64_t stream);            /* back to 0 after a reported failure was handled */
/* The same word copied to (pinned) host memory in stream order, without waiting: a host that already waits
 * for an event later on that stream reads it then. */
int qmoe_device_status_async(uint64_t stream, void* host_status);

/* Test hook (no upstream counterpart): selects, process-wide, the comparison form of a kernel that the
 * parity tests run against the default form.  value 0 = default, 1 = comparison form.  Not for production
 * hosts: the defaults are the measured-faster forms. */
enum {
    QMOE_VARIANT_SINGLE_CTA_GEMM = 0,   /* expert GEMMs with one CTA per 128 x 256 tile instead of a CTA pair per 256 x 256 */
    QMOE_VARIANT_WGRAD_PER_PRODUCT = 1, /* one launch per weight-gradient product instead of one for all three */
    QMOE_VARIANT_NARROW_SCATTER = 2,    /* 64-byte instead of 256-byte row pieces in the peer-memory scatter epilogues */
    QMOE_VARIANT_PLAIN_GEMM_ON_CUDA_CORES = 3, /* qmoe_gemm never takes the tensor-core kernels */
    QMOE_VARIANT_COUNT = 4
};
int qmoe_test_select_variant(int32_t which, int32_t value);

/* ---------------------------------------------------------------------------------------------
 * Sizes
 * ------------------------------------------------------------------------------------------- */
/* Upper bound of rows in the dispatched layout: A + E*(QMOE_ROW_PAD-1), rounded up to the pad. */
int64_t qmoe_rows_bound(int64_t tokens, int32_t experts, int32_t top_k);
/* Blocks the routing kernels use for T tokens (first dimension of the block_* scratch tables). */
int64_t qmoe_route_blocks(int64_t tokens);

/* ---------------------------------------------------------------------------------------------
 * Routing tables (caller-allocated; the struct only carries addresses)
 * ------------------------------------------------------------------------------------------- */
typedef struct qmoe_route {
    int64_t tokens;        /* T */
    int32_t experts;       /* E  (<= QMOE_MAX_EXPERTS) */
    int32_t top_k;         /* k  (<= min(E, QMOE_MAX_TOP_K)) */
    int64_t rows_bound;    /* qmoe_rows_bound(T, E, k) */
    uint64_t probs;        /* f32 [T, E]   softmax of the scores */
    uint64_t gate_weights; /* f32 [T, k]   renormalised gate weights, slot order = descending prob */
    uint64_t expert_index; /* i32 [A]      expert of assignment a = token*k + slot */
    uint64_t dest_row;     /* i32 [A]      row of assignment a in the dispatched layout */
    uint64_t row_source;   /* i32 [rows_bound]  assignment held by each dispatched row, -1 = pad */
    uint64_t counts;       /* i32 [E]      rows routed to each expert */
    uint64_t offsets;      /* i32 [E + 1]  first dispatched row of each expert (multiples of the pad) */
    uint64_t tile_expert;  /* i32 [rows_bound / QMOE_ROW_PAD]  expert owning each 128-row tile */
    uint64_t meta;         /* i32 [4]      {dispatched rows incl. pads, 128-row tiles, A, 0} */
    uint64_t utilization;  /* f32 [E]      counts / A */
    uint64_t aux;          /* f32 [1]      load-balancing loss */
    uint64_t block_counts; /* i32 [blocks, E]  scratch */
    uint64_t block_base;   /* i32 [blocks, E]  scratch */
    uint64_t block_colsum; /* f32 [blocks, E]  scratch */
} qmoe_route_t;

/* Router logits: scores[T, E] = float(x)[T, d] . w_router[E, d]^T in fp32 semantics whatever the
 * activation dtype.  Replaces the router `linear` call under `set_matmul_precision(None)`
 * (src/qutai/lm/layers.py:377-378, gemm kernels src/qutai/backends/cuda/gemm.cu:35-101).
 * With bf16 activations, at most 64 experts and a scratch buffer of qmoe_router_scratch_bytes(T, E, d)
 * bytes (256-byte aligned) the product runs on the tensor cores with the fp32 weights split into three
 * bf16 terms (exact products, fp32 accumulation); otherwise on the CUDA cores.  qmoe_router_logits is
 * the scratch-free form. */
int64_t qmoe_router_scratch_bytes(int64_t tokens, int32_t experts, int64_t width);
int qmoe_router_forward(uint64_t x, int32_t x_dtype, uint64_t w_router, uint64_t scores, uint64_t scratch,
                        int64_t tokens, int64_t width, int32_t experts, uint64_t stream);
int qmoe_router_logits(uint64_t x, int32_t x_dtype, uint64_t w_router, uint64_t scores,
                       int64_t tokens, int64_t width, int32_t experts, uint64_t stream);
/* Router backward: dx_router[T, d] (f32) = d_scores . w_router ; d_w_router[E, d] (f32) =
 * d_scores^T . float(x), deterministic (token blocks reduced in a fixed order).  `scratch` as above
 * (qmoe_router_grad_partials gives the same size in 4-byte units).  Replaces the backward closure
 * of `linear` (src/qutai/lm/layers.py:50-70) for the router. */
int64_t qmoe_router_grad_partials(int64_t tokens, int32_t experts, int64_t width);
int qmoe_router_backward(uint64_t d_scores, uint64_t x, int32_t x_dtype, uint64_t w_router,
                         uint64_t dx_router, uint64_t d_w_router, uint64_t scratch,
                         int64_t tokens, int64_t width, int32_t experts, uint64_t stream);

/* Softmax, top-k (ties -> lowest expert index), gate renormalisation, per-expert counts, padded
 * offsets, the stable dispatch permutation, utilisation and the auxiliary loss, all on the device
 * and without a host synchronisation.  Replaces `routing` (src/qutai/backends/cuda_lm.py:368-449:
 * softmax, lm_route, lm_route_pack, lm_route_util, lm_route_aux; CPU statement
 * src/qutai/backends/cpu_lm.py:204-242). */
int qmoe_route(const qmoe_route_t* route, uint64_t scores, uint64_t stream);
/* qmoe_route for callers that cannot allocate device memory for its three scratch tables (a
 * serving loop that must not call cudaMalloc on its request path, a plug-in host limited to the
 * buffers it was given at start-up): route->block_counts, block_base and block_colsum are ignored
 * and a 1.5 MiB array built into the library is used instead.  Limit: qmoe_route_blocks(tokens) *
 * experts <= 131072, otherwise an argument error.  Allocates nothing.  The array is shared by all
 * calls on a device, so calls that overlap on the GPU race: use one stream at a time.  The first
 * call on a device resolves the array's address and should be made before any stream capture.
 * The filled route can be handed to every other entry point with the three scratch fields left 0
 * (only qmoe_route itself needs them); qmoe_ep_pack_stats / qmoe_ep_gather_stats, which read the
 * column sums out of block_colsum, reject such a route.
 * This entry point has no counterpart in the upstream project. */
int qmoe_route_static(const qmoe_route_t* route, uint64_t scores, uint64_t stream);
/* The same tables in the upstream layout, for hosts that keep the upstream `route` dict
 * (src/qutai/backends/cuda_lm.py:435-449): int64 indices[A], ids[E*capacity], slots[E*capacity]
 * (row e holds expert e's token rows / slot numbers), locations[A], counts[E]. */
int qmoe_route_export_i64(const qmoe_route_t* route, uint64_t indices, uint64_t ids, uint64_t slots,
                          uint64_t locations, uint64_t counts, int64_t capacity, uint64_t stream);
/* d_scores[T, E] (f32) = gate-weight path (grad_weights f32 [T, k], may be 0) + auxiliary-loss path
 * (grad_aux f32 [1], may be 0).  Replaces the two `routing_backward` calls and the add that joins
 * them (src/qutai/backends/cuda_lm.py:452-468, src/qutai/backends/cuda/lm.cu:388-393,
 * src/qutai/backends/cpu_lm.py:245-276). */
int qmoe_route_backward(const qmoe_route_t* route, uint64_t grad_weights, uint64_t grad_aux,
                        uint64_t d_scores, uint64_t stream);

/* ---------------------------------------------------------------------------------------------
 * Permute / combine (memory-bound, 128-bit accesses when the row pitch allows)
 * ------------------------------------------------------------------------------------------- */
/* dispatched[r, :] = x[token(r), :], pad rows zero.  Replaces the E `route_gather` launches
 * (src/qutai/backends/cuda_lm.py:471-485, src/qutai/backends/cuda/lm.cu:394-396). */
int qmoe_permute(const qmoe_route_t* route, uint64_t x, uint64_t dispatched, int32_t dtype,
                 int64_t width, uint64_t stream);
/* dx[t, :] = sum_s d_dispatched[dest_row(t, s), :] (+ extra_f32[t, :] when extra != 0), summed in
 * fp32 and rounded once.  Replaces `route_gather_backward` (E zero-filled T x d buffers,
 * src/qutai/backends/cuda_lm.py:488-502) and the pairwise adds of src/qutai/core/grad.py:62. */
int qmoe_unpermute_reduce(const qmoe_route_t* route, uint64_t d_dispatched, uint64_t extra_f32,
                          uint64_t dx, int32_t dtype, int64_t width, uint64_t stream);
/* out[t, :] = sum_s gate_weights[t, s] * y_dispatched[dest_row(t, s), :], fp32 sum, one rounding.
 * Replaces `combine` (src/qutai/backends/cuda_lm.py:521-541, lm_combine_all lm.cu:406-416). */
int qmoe_combine(const qmoe_route_t* route, uint64_t y_dispatched, uint64_t out, int32_t dtype,
                 int64_t width, uint64_t stream);
/* dy_dispatched[r, :] = g[token(r), :] * w(r) (pad rows zero); d_gate_weights[a] (f32) =
 * <g[token, :], y_dispatched[r, :]>.  Replaces `combine_backward`
 * (src/qutai/backends/cuda_lm.py:544-581, lm.cu:417-429). */
int qmoe_combine_backward(const qmoe_route_t* route, uint64_t grad_out, uint64_t y_dispatched,
                          uint64_t dy_dispatched, uint64_t d_gate_weights, int32_t dtype,
                          int64_t width, uint64_t stream);

/* ---------------------------------------------------------------------------------------------
 * Expert FFN (grouped GEMMs)
 * ------------------------------------------------------------------------------------------- */
typedef struct qmoe_experts {
    int32_t experts;   /* E */
    int32_t dtype;     /* activation dtype: QMOE_BF16 -> bf16 operands, fp32 accumulate (tcgen05);
                          QMOE_F32 -> fp32 everywhere (CUDA cores) */
    int32_t engine;    /* QMOE_ENGINE_* ; AUTO = tcgen05 whenever dtype is bf16 and d, h are multiples of 8 */
    int32_t reserved;
    int64_t width;     /* d */
    int64_t hidden;    /* h */
    /* stacked expert weights in the OPERAND dtype (bf16 shadows for QMOE_BF16, the fp32 masters
     * for QMOE_F32): gate, up [E, h, d]; down [E, d, h]  (upstream `Projection.weight` is
     * (outputs, inputs), src/qutai/lm/layers.py:260-266) */
    uint64_t w_gate, w_up, w_down;
} qmoe_experts_t;

/* fp32 -> bf16 (round to nearest even) of n elements: refreshes the bf16 operand copies of the
 * fp32 master weights.  Upstream rounds the same way while staging tiles
 * (src/qutai/backends/cuda/gemm.cu:23-24, :122-127). */
int qmoe_cast_bf16(uint64_t src_f32, uint64_t dst_bf16, int64_t n, uint64_t stream);

/* For every expert group of the dispatched input X:  G = X Wg^T, U = X Wu^T, H = silu(G) * U,
 * Y = H Wd^T.  G, U, H are [rows_bound, h]; X, Y are [rows_bound, d].  Replaces the per-expert
 * `SwiGLU.__call__` (src/qutai/lm/layers.py:310-311: 3 gemm + lm_silu + multiply per expert). */
int qmoe_expert_forward(const qmoe_route_t* route, const qmoe_experts_t* experts, uint64_t x_dispatched,
                        uint64_t g, uint64_t u, uint64_t h, uint64_t y_dispatched, uint64_t stream);
/* The same forward in two parts, for hosts that pipeline it with an exchange: QMOE_FWD_UP computes
 * G, U, H; QMOE_FWD_DOWN computes Y from H.  Both bits = qmoe_expert_forward. */
enum { QMOE_FWD_UP = 1, QMOE_FWD_DOWN = 2 };
int qmoe_expert_forward_parts(const qmoe_route_t* route, const qmoe_experts_t* experts, uint64_t x_dispatched,
                              uint64_t g, uint64_t u, uint64_t h, uint64_t y_dispatched, int32_t parts,
                              uint64_t stream);
/* Backward of the above.  dH (scratch [rows_bound, h]), dG, dU [rows_bound, h]; dX [rows_bound, d];
 * d_w_gate, d_w_up [E, h, d] and d_w_down [E, d, h] are fp32 and are WRITTEN (not accumulated) for
 * experts that received rows and left untouched for the others (upstream such experts get no
 * gradient at all, src/qutai/lm/layers.py:396).  Replaces the closures of
 * src/qutai/lm/layers.py:50-70, :104 and src/qutai/core/operations/elementwise.py:44-51. */
int qmoe_expert_backward(const qmoe_route_t* route, const qmoe_experts_t* experts,
                         uint64_t dy_dispatched, uint64_t x_dispatched, uint64_t g, uint64_t u,
                         uint64_t h, uint64_t d_h, uint64_t d_g, uint64_t d_u, uint64_t dx_dispatched,
                         uint64_t d_w_gate, uint64_t d_w_up, uint64_t d_w_down, uint64_t stream);

/* The same backward in two parts, for hosts that overlap an exchange with the weight gradients:
 * QMOE_BWD_ACTIVATIONS computes dG, dU and dX (dX must then have its own buffer, not dY's),
 * QMOE_BWD_WEIGHTS the three weight gradients.  Both bits = qmoe_expert_backward. */
enum { QMOE_BWD_ACTIVATIONS = 1, QMOE_BWD_WEIGHTS = 2,
       QMOE_BWD_NO_DX = 4 /* with ACTIVATIONS: leave dX out (the caller computes it with qmoe_ep_expert_dx_push) */ };
int qmoe_expert_backward_parts(const qmoe_route_t* route, const qmoe_experts_t* experts,
                               uint64_t dy_dispatched, uint64_t x_dispatched, uint64_t g, uint64_t u,
                               uint64_t h, uint64_t d_h, uint64_t d_g, uint64_t d_u, uint64_t dx_dispatched,
                               uint64_t d_w_gate, uint64_t d_w_up, uint64_t d_w_down, int32_t parts,
                               uint64_t stream);

/* Plain (single-group) product C[M, N] = op(A) op(B) with the upstream dispatcher's meaning of
 * the arguments (src/qutai/backends/cuda.py:305-362): A is [M, K] ([K, M] when transpose_a),
 * B is [K, N] ([N, K] when transpose_b); dtypes per operand; accumulate adds into C.  Like upstream's
 * dispatcher (:346-355) it picks a kernel by shape and dtype: bf16 x bf16 without accumulate runs on the
 * tcgen05 kernels when the sizes are multiples of 8 and the addresses of 16 bytes — A . B^T and A . B with a
 * bf16 result and M a multiple of 128, A^T . B with an fp32 result (a weight gradient); everything else on
 * the CUDA cores. */
int qmoe_gemm(uint64_t a, int32_t a_dtype, uint64_t b, int32_t b_dtype, uint64_t c, int32_t c_dtype,
              int64_t m, int64_t k, int64_t n, int32_t transpose_a, int32_t transpose_b,
              int32_t accumulate, uint64_t stream);
/* The weight gradient of a linear layer, C[M, N] (fp32) = A^T . B with A [K, M] and B [K, N] in bf16 (qmoe_gemm with
 * transpose_a), for shapes whose few 256 x 256 tiles would leave most of the GPU idle: the K rows are cut into ranges
 * that run side by side on the tcgen05 kernels, each into a slab of `partials`, and the slabs are added in a fixed
 * order (bit-identical from run to run).  `partials`: qmoe_gemm_wgrad_partials(m, k, n) 4-byte units, 16-byte aligned;
 * that function gives 0 when the shape is not split, and qmoe_gemm is the call to make then.  Upstream has one product
 * for this (the backward closure of `linear`, src/qutai/lm/layers.py:260-272). */
int64_t qmoe_gemm_wgrad_partials(int64_t m, int64_t k, int64_t n);
int qmoe_gemm_wgrad_split(uint64_t a, uint64_t b, uint64_t c, uint64_t partials, int64_t m, int64_t k, int64_t n,
                          uint64_t stream);
/* silu(v) (backward == 0) or g * silu'(v) (backward != 0), element-wise over n values.
 * Replaces lm_silu (src/qutai/backends/cuda/lm.cu:54). */
int qmoe_silu(uint64_t values, uint64_t gradient, uint64_t out, int32_t dtype, int64_t n,
              int32_t backward, uint64_t stream);

/* out = a + b element-wise (the sum autograd applies when a tensor receives several gradient
 * contributions, src/qutai/core/grad.py:62, and when a leaf accumulates, src/qutai/core/tensor.py:207-209). */
int qmoe_add(uint64_t a, uint64_t b, uint64_t out, int32_t dtype, int64_t n, uint64_t stream);
/* dst[i, :] = src[index[i], :] for i < rows (index: i32 on the device, entries in [0, src_rows); row_bytes a
 * multiple of 4).  Used for the small expert-indexed tables (router weight rows, their gradient, utilisation)
 * when the expert-parallel layer places experts on ranks by a map instead of by contiguous blocks; upstream
 * has one device and no such map. */
int qmoe_gather_rows(uint64_t src, uint64_t dst, uint64_t index, int32_t rows, int32_t src_rows, int64_t row_bytes,
                     uint64_t stream);
/* Fill n values with N(mean, std) from a counter-based generator keyed by (seed, index).  Plays
 * the role of `normal` (src/qutai/backends/cuda_lm.py:27-28, normal_fill
 * src/qutai/backends/cuda/gemm.cu:146-161); like upstream, the stream differs from the CPU
 * generator's for the same seed, so parity tests copy weights instead of comparing draws. */
int qmoe_normal_fill(uint64_t out, int32_t dtype, int64_t n, double mean, double std, uint64_t seed,
                     uint64_t stream);

/* ---------------------------------------------------------------------------------------------
 * Whole layer in one call (removes the per-stage host round trips; same kernels as above)
 * ------------------------------------------------------------------------------------------- */
typedef struct qmoe_layer {
    qmoe_route_t route;
    qmoe_experts_t experts;
    uint64_t x;            /* [T, d] activations (experts.dtype) */
    uint64_t w_router;     /* f32 [E, d] */
    uint64_t scores;       /* f32 [T, E] */
    uint64_t x_dispatched, g, u, h, y_dispatched;   /* saved for the backward */
    uint64_t out;          /* [T, d] */
    /* backward */
    uint64_t grad_out;     /* [T, d] */
    uint64_t grad_aux;     /* f32 [1] or 0 */
    uint64_t dy_dispatched, d_h, d_g, d_u, dx_dispatched;  /* dx_dispatched may alias dy_dispatched */
    uint64_t d_gate_weights; /* f32 [T, k] */
    uint64_t d_scores;     /* f32 [T, E] */
    uint64_t dx_router;    /* f32 [T, d] */
    uint64_t router_partials;
    uint64_t dx;           /* [T, d] */
    uint64_t d_w_router;   /* f32 [E, d] */
    uint64_t d_w_gate, d_w_up, d_w_down; /* f32 stacked */
    /* fp32 master weights to refresh the bf16 operand copies from before the forward (0 = skip) */
    uint64_t master_gate, master_up, master_down;
} qmoe_layer_t;

/* Forward of `SparseMoE.__call__` (src/qutai/lm/layers.py:376-402): router logits, routing,
 * permute, grouped expert FFN, weighted combine. */
int qmoe_layer_forward(const qmoe_layer_t* layer, uint64_t stream);
/* Backward of the same call (the closures listed above, in the order src/qutai/core/grad.py:34-65
 * would run them), producing dx, d_w_router and the stacked expert weight gradients. */
int qmoe_layer_backward(const qmoe_layer_t* layer, uint64_t stream);

/* ---------------------------------------------------------------------------------------------
 * The step either side of the layer inside a decoder block, fused into the layer's first read and last write:
 *     out = x + MoE(rms_norm(x, w))
 * Upstream: Block.__call__ (src/qutai/lm/layers.py:430-437) = residual_add(x, ffn(ffn_norm(x))), rms_norm
 * src/qutai/lm/layers.py:88-96, kernels lm_rms / lm_rms_dx / lm_rms_dw src/qutai/backends/cuda/lm.cu:40-53 (launched
 * from src/qutai/backends/cuda_lm.py:124-178; the norm's output is an fp32 copy of the activations there), CPU
 * statement src/qutai/backends/cpu_lm.py:84-117.  rms_norm(x, w)[t, j] = x[t, j] * inverse[t] * w[j] with
 * inverse[t] = 1 / sqrt(mean_j x[t, j]^2 + eps); w is f32 [d].
 * ------------------------------------------------------------------------------------------- */
/* inverse[t] (f32 [T]) of every token row: the statistic half of lm_rms; the normalised activations themselves
 * are never written. */
int qmoe_rms_inverse(uint64_t x, int32_t dtype, uint64_t inverse, int64_t tokens, int64_t width, double eps,
                     uint64_t stream);
/* out[r, c] = in[r, c] * row_scale[r] * col_scale[c] (f32; either scale may be 0 = none; in place allowed).  Folds
 * the norm weight into the router weight (columns), applies inverse[t] to the logits of the raw activations (rows),
 * and the reverse for the router's gradients. */
int qmoe_scale_f32(uint64_t in, uint64_t out, uint64_t row_scale, uint64_t col_scale, int64_t rows, int64_t cols,
                   uint64_t stream);
/* qmoe_permute with the norm applied to the row it copies: dispatched[r, :] = round(x[token(r), :] * inverse[token] * w). */
int qmoe_permute_norm(const qmoe_route_t* route, uint64_t x, uint64_t inverse, uint64_t norm_weight, uint64_t dispatched,
                      int32_t dtype, int64_t width, uint64_t stream);
/* qmoe_combine with the residual added before the single rounding: out[t, :] = round(residual[t, :] + sum_s w y). */
int qmoe_combine_residual(const qmoe_route_t* route, uint64_t y_dispatched, uint64_t residual, uint64_t out, int32_t dtype,
                          int64_t width, uint64_t stream);
/* qmoe_unpermute_reduce with the norm's backward (lm_rms_dx, lm_rms_dw) and the residual's gradient folded in.  With
 * d_n[t] = sum_s d_dispatched[dest_row(t, s)] + extra_f32[t] (gradient of the normalised input; extra may be 0;
 * with extra_row_scaled != 0 the buffer holds inverse[t] * addend and the kernel divides the row scale out):
 *   dx[t, j] = round(grad_out[t, j] + inverse[t] * (d_n[j] w[j] - x[t, j] inverse[t]^2 mean_j(d_n[j] w[j] x[t, j])))
 *   d_norm_weight[j] (f32 [d], written) = sum_t d_n[t, j] x[t, j] inverse[t], reduced in a fixed order.
 * partials: scratch of qmoe_norm_backward_partials(T, d) floats.  width <= 4096, else QMOE_ERR_UNSUPPORTED. */
int64_t qmoe_norm_backward_partials(int64_t tokens, int64_t width);
int qmoe_unpermute_norm_backward(const qmoe_route_t* route, uint64_t d_dispatched, uint64_t extra_f32,
                                 int32_t extra_row_scaled, uint64_t x, uint64_t inverse, uint64_t norm_weight,
                                 uint64_t grad_out, uint64_t dx, uint64_t d_norm_weight, uint64_t partials, int32_t dtype,
                                 int64_t width, uint64_t stream);
/* The whole feed-forward half of a block in one call per direction: layer.out = layer.x + MoE(rms_norm(layer.x)),
 * and its backward (layer.dx = gradient of layer.x including the residual's, d_norm_weight written).  `layer` is
 * filled as for qmoe_layer_forward / qmoe_layer_backward; layer.out must not alias layer.x. */
typedef struct qmoe_block {
    qmoe_layer_t layer;
    uint64_t norm_weight;      /* f32 [d] */
    uint64_t inverse;          /* f32 [T]      written by the forward, read by the backward */
    uint64_t w_router_folded;  /* f32 [E, d]   scratch: router weight times the norm weight */
    uint64_t d_norm_weight;    /* f32 [d]      backward output */
    uint64_t norm_partials;    /* f32 [qmoe_norm_backward_partials(T, d)] scratch */
    double norm_eps;
} qmoe_block_t;
int qmoe_block_forward(const qmoe_block_t* block, uint64_t stream);
int qmoe_block_backward(const qmoe_block_t* block, uint64_t stream);

/* ---------------------------------------------------------------------------------------------
 * The language-model head and its cross-entropy loss (the caller after the last block):
 *     loss = mean over counted rows r of  log sum_c exp(z[r, c]) - z[r, label(r)],   z = rows(hidden) . weight^T
 * where the rows are every position but the last of each sequence and label(r) is the token that follows it
 * (-100, like any value outside [0, vocab), = not counted; the mean divides by max(1, counted rows)).  Replaces `projection_loss`
 * (src/qutai/lm/layers.py:187-257) with its lm_head_rows / gemm / lm_head_loss / lm_head_gradient launches per
 * chunk (src/qutai/backends/cuda_lm.py, kernels src/qutai/backends/cuda/lm.cu:430-444; CPU statement
 * src/qutai/backends/cpu_lm.py:323-371).  The logits of all rows are formed once and kept: the forward leaves the
 * loss and, in place of the logits, their gradient for an incoming gradient of 1; the backward is the two
 * remaining products.  dtype QMOE_BF16 (bf16 hidden, bf16 weight operand, bf16 logits: tcgen05 when width and vocab
 * are multiples of 8) or QMOE_F32 (CUDA cores).
 * ------------------------------------------------------------------------------------------- */
typedef struct qmoe_head {
    int32_t batch, time;       /* hidden is [batch, time, width]; head rows = batch * (time - 1) */
    int32_t dtype;             /* QMOE_BF16 / QMOE_F32: hidden, weight, inputs, logits, d_inputs, d_hidden */
    int32_t reserved;
    int64_t width, vocab;
    int64_t rows_bound;        /* head rows rounded up to a multiple of 128: row count of inputs, logits, d_inputs */
    uint64_t hidden;           /* [batch * time, width] */
    uint64_t weight;           /* [vocab, width] */
    uint64_t labels;           /* i64 [batch, time] token ids; the label of position t is labels[b, t + 1] */
    uint64_t inputs;           /* [rows_bound, width]  the gathered rows (kept for the backward) */
    uint64_t logits;           /* [rows_bound, vocab]  logits, overwritten by their gradient */
    uint64_t row_loss;         /* f32 [rows] */
    uint64_t loss;             /* f32 [1] */
    uint64_t meta;             /* 32 bytes scratch, 16-byte aligned: 1 / count and the one group of the products */
    uint64_t d_inputs;         /* [rows_bound, width] scratch of the backward (0 with d_hidden == 0) */
    uint64_t d_hidden;         /* [batch * time, width], every row written (the last positions zero); 0 = not wanted */
    uint64_t d_weight;         /* f32 [vocab, width], overwritten; 0 = not wanted */
} qmoe_head_t;
int qmoe_head_forward(const qmoe_head_t* head, uint64_t stream);
/* gradient: f32 [1] on the device, the gradient of whatever follows with respect to the loss; 0 = 1.0 */
int qmoe_head_backward(const qmoe_head_t* head, uint64_t gradient, uint64_t stream);
/* The per-chunk functions of the upstream backend table, for hosts that keep its chunked loop
 * (src/qutai/backends/cuda_lm.py:584-660, src/qutai/lm/layers.py:199-255).  `labels`: i64 targets, one per head row (the
 * upstream prepared labels); rows [start, start + rows) are the chunk.
 * qmoe_head_rows: out[i, :] = values[position(start + i), :], or with backward != 0 out[position(start + i), :] += values[i, :]
 *   (position(r) = (r / (time - 1)) * time + r % (time - 1));
 * qmoe_head_loss: out[0] (f32) = sum over the chunk's counted rows of log sum exp - picked logit (row_loss: f32 [rows] scratch);
 * qmoe_head_gradient: logits[r, :] <- gradient[0] / count * (softmax - one_hot), zero for rows that are not counted
 *   (factor: f32 [1] scratch). */
int qmoe_head_rows(uint64_t values, uint64_t out, int32_t dtype, int64_t start, int64_t count, int64_t width,
                   int64_t time, int32_t backward, uint64_t stream);
int qmoe_head_loss(uint64_t logits, int32_t dtype, uint64_t labels, uint64_t row_loss, uint64_t out, int64_t rows,
                   int64_t vocab, int64_t start, uint64_t stream);
int qmoe_head_gradient(uint64_t logits, int32_t dtype, uint64_t labels, uint64_t gradient, uint64_t factor, int64_t count,
                       int64_t rows, int64_t vocab, int64_t start, uint64_t stream);

/* ---------------------------------------------------------------------------------------------
 * The small operations around attention and the feed-forward half of a block, with the upstream launchers' meaning of
 * the arguments (src/qutai/backends/cuda_lm.py:77-228, kernels src/qutai/backends/cuda/lm.cu:11-64, CPU statements
 * src/qutai/backends/cpu_lm.py:54-140).  Weights are f32; activations f32 or bf16 per argument.
 * ------------------------------------------------------------------------------------------- */
/* out[r, :] = x[r, :] * inverse[r] * weight, inverse[r] (f32) = 1 / sqrt(mean(x[r, :]^2) + eps).  Replaces `rms_norm` (lm_rms). */
int qmoe_rms_norm(uint64_t x, int32_t x_dtype, uint64_t weight, uint64_t out, int32_t out_dtype, uint64_t inverse,
                  int64_t rows, int64_t width, double eps, uint64_t stream);
/* dx (dtype of x) and d_weight (f32 [width], overwritten; summed over rows in a fixed order).  `partials`: f32 scratch of
 * qmoe_rms_norm_partials(rows, width) elements.  Replaces `rms_norm_backward` (lm_rms_dx, lm_rms_dw). */
int64_t qmoe_rms_norm_partials(int64_t rows, int64_t width);
int qmoe_rms_norm_backward(uint64_t gradient, int32_t g_dtype, uint64_t x, int32_t x_dtype, uint64_t weight,
                           uint64_t inverse, uint64_t dx, uint64_t d_weight, uint64_t partials, int64_t rows,
                           int64_t width, uint64_t stream);
/* Rotary position embedding of [batch, time, heads, dim]: pairs (2 i, 2 i + 1) turned by (offset + t) theta^(-2 i / dim),
 * the other way round with inverse != 0 (its own backward).  Replaces `rope` (lm_rope). */
int qmoe_rope(uint64_t values, uint64_t out, int32_t dtype, int64_t batch, int64_t time, int32_t heads, int32_t dim,
              double theta, int32_t offset, int32_t inverse, uint64_t stream);
/* out[i, :] = weight[ids[i], :] (ids i64; an id outside [0, vocab) gives a zero row).  Replaces `embedding` (lm_embedding). */
int qmoe_embedding(uint64_t weight, uint64_t ids, uint64_t out, int32_t out_dtype, int64_t count, int64_t width,
                   int64_t vocab, uint64_t stream);
/* d_weight[tokens[s], :] += sum of gradient[p, :] over positions[starts[s] .. starts[s + 1]), in that order (i64 tables made
 * on the host as upstream makes them: distinct tokens ascending, each with its positions ascending).  d_weight f32
 * [vocab, width] is added to: zero it first for upstream's `embedding_backward` (lm_embedding_backward). */
int qmoe_embedding_backward(uint64_t gradient, int32_t g_dtype, uint64_t tokens, uint64_t starts, uint64_t positions,
                            uint64_t d_weight, int64_t segments, int64_t count, int64_t width, int64_t vocab,
                            uint64_t stream);

/* ---------------------------------------------------------------------------------------------
 * Causal self-attention with grouped key/value heads (the other half of a decoder block):
 *     out[b, t, h, :] = sum_{s <= t} softmax_s(q[b, t, h, :] . k[b, s, h / (heads / kv_heads), :] / sqrt(dim)) v[b, s, ..., :]
 * and its backward.  Replaces `attention` / `attention_backward` (src/qutai/lm/layers.py:119-130, launchers
 * src/qutai/backends/cuda_lm.py, kernels lm_attention_bf16_d64 / _dq / _dkv src/qutai/backends/cuda/lm.cu:91-285;
 * CPU statement src/qutai/backends/cpu_lm.py:141-201).  Head width 64 and bf16 only (the upstream tensor-core
 * kernels' case), any sequence length; tcgen05, the time x time scores are never written.
 * ------------------------------------------------------------------------------------------- */
typedef struct qmoe_attention {
    int32_t batch, time, heads, kv_heads;
    int32_t dim;               /* 64 */
    int32_t dtype;             /* QMOE_BF16 */
    uint64_t q;                /* [batch, time, heads, dim] */
    uint64_t k, v;             /* [batch, time, kv_heads, dim] */
    uint64_t out;              /* [batch, time, heads, dim] */
    uint64_t lse;              /* f32 [batch, time, heads]: log sum exp of the scaled scores of every row */
    uint64_t grad_out;         /* backward: gradient of out */
    uint64_t delta;            /* backward: f32 [batch, time, heads] scratch */
    uint64_t dq, dk, dv;       /* backward: like q, k, v */
} qmoe_attention_t;
int qmoe_attention_forward(const qmoe_attention_t* attention, uint64_t stream);
/* needs q, k, v, out and lse as the forward left them */
int qmoe_attention_backward(const qmoe_attention_t* attention, uint64_t stream);

/* ---------------------------------------------------------------------------------------------
 * Expert parallelism (one process per GPU, NCCL over NVLink / NVSwitch).  The upstream project is
 * single-GPU (src/qutai/backends/cuda_runtime.py:82, :105), so these entry points have no upstream
 * counterpart; they keep the layer's semantics when tokens are sharded T/N per rank (contiguous
 * shards) and experts E/N per rank (contiguous blocks): an expert's rows arrive ordered by source
 * rank, which is the upstream global (token, slot) order (src/qutai/backends/cuda/lm.cu:353-383),
 * and utilisation / auxiliary loss are computed over all ranks' tokens
 * (src/qutai/backends/cpu_lm.py:221-229).
 * ------------------------------------------------------------------------------------------- */
typedef struct qmoe_ep_segment {
    int32_t peer;          /* rank on the other side */
    int32_t reserved;
    int64_t offset_rows;   /* first row of the segment in the local buffer */
    int64_t rows;          /* rows to move (0 = skipped on both sides) */
} qmoe_ep_segment_t;

/* Rank 0 creates a 128-byte id and hands it to every rank by any host channel; every rank then
 * calls qmoe_ep_init with its device current.  One communicator per process. */
int qmoe_ep_unique_id(void* id128);
int qmoe_ep_init(int32_t rank, int32_t world, const void* id128);
/* abort_communicator != 0 tears the communicator down without waiting for outstanding work (the
 * path to take after the host learned that a peer is gone). */
int qmoe_ep_finalize(int32_t abort_communicator);
int qmoe_ep_info(int32_t* rank, int32_t* world);
/* After qmoe_route on the local tokens: pack {counts[E], probability column sums[E] (float bits)}
 * into stats_local (i32 [2E]), all-gather into stats_all (i32 [world, 2E]) and, when host_stats is
 * not null, start its copy to (pinned) host memory; synchronise the stream before reading it. */
int qmoe_ep_gather_stats(const qmoe_route_t* route, uint64_t stats_local, uint64_t stats_all,
                         void* host_stats, uint64_t stream);
/* From stats_all: overwrite token_route->utilization and ->aux with the values over all ranks'
 * tokens, and fill expert_route's counts / offsets / tile_expert / meta for this rank's
 * E / world experts (rows of all ranks, padded like the single-GPU dispatched layout). */
int qmoe_ep_plan(uint64_t stats_all, const qmoe_route_t* token_route, const qmoe_route_t* expert_route,
                 int64_t tokens_global, uint64_t stream);
/* Zero the pad rows of every expert group of a buffer in expert_route's dispatched layout. */
int qmoe_ep_zero_pad_rows(const qmoe_route_t* expert_route, uint64_t buffer, int32_t dtype,
                          int64_t width, uint64_t stream);
/* One grouped exchange: every send segment [offset_rows, +rows) of send_buffer goes to its peer,
 * every receive segment of recv_buffer is filled from its peer.  Between a pair of ranks segments
 * are matched in list order.  This is the dispatch / combine all-to-all(v). */
int qmoe_ep_exchange(uint64_t send_buffer, const qmoe_ep_segment_t* sends, int32_t n_sends,
                     uint64_t recv_buffer, const qmoe_ep_segment_t* recvs, int32_t n_recvs,
                     int64_t width, int32_t dtype, uint64_t stream);
/* In-place sum over ranks (router weight gradient). */
int qmoe_ep_all_reduce_f32(uint64_t buffer, int64_t n, uint64_t stream);

/* Direct transport over peer memory (no upstream counterpart).  Instead of NCCL send/receive, rows
 * are pushed into the destination rank's buffer with plain stores over NVLink; destinations are
 * computed on the device from the gathered counts, so the host does not read them.  Buffers that
 * other ranks write into must come from one cudaMalloc each (qmoe_malloc), are exported with
 * qmoe_ep_ipc_export, and opened by every other rank with qmoe_ep_ipc_open (all GPUs of the job
 * must be visible to every process).  After a push, qmoe_ep_barrier (NCCL) or qmoe_ep_flag_barrier
 * (flags in peer memory; the one kernel that waits on another GPU, for a bounded time) orders it against
 * the readers on every rank. */
#define QMOE_EP_MAX_RANKS 16
typedef struct qmoe_ep_peers {
    int32_t world;
    int32_t rank;
    uint64_t buffer[QMOE_EP_MAX_RANKS]; /* the same buffer on every rank (own entry: local address) */
    uint64_t ret[QMOE_EP_MAX_RANKS];    /* i32 return-address table of every rank (dispatch only) */
} qmoe_ep_peers_t;
int qmoe_set_device(int32_t device);
int qmoe_ep_ipc_export(uint64_t address, void* handle64);
int qmoe_ep_ipc_open(const void* handle64, uint64_t* address);
int qmoe_ep_ipc_close(uint64_t address);
/* A 1-element all-reduce on scratch_i32: when it has run on a rank, every rank has finished the
 * work it enqueued before its own call. */
int qmoe_ep_barrier(uint64_t scratch_i32, uint64_t stream);
/* dest_base[e] (i32 [E]) = row, in the expert-side layout of the rank owning expert e, where this
 * rank's rows for e start (after the rows of lower ranks). */
int qmoe_ep_dest_base(uint64_t stats_all, int32_t experts, int32_t local_experts, uint64_t dest_base,
                      uint64_t stream);
/* Token side -> expert side: every real row of `src` (local dispatched layout of token_route) is
 * stored into the owner's buffer; with write_return_addresses the owner's return table gets
 * (source rank, source row) for each row.  blocks_per_sm: 0 = use the whole GPU; 1 = small enough
 * to run beside a tensor-core kernel on every SM (for pushes issued on a second stream). */
int qmoe_ep_push_dispatch(const qmoe_route_t* token_route, uint64_t dest_base, uint64_t src,
                          const qmoe_ep_peers_t* peers, int32_t write_return_addresses,
                          int32_t blocks_per_sm, int32_t dtype, int64_t width, uint64_t stream);
/* Expert side -> token side: every real row of `src` (expert-side layout) that belongs to a local
 * expert in [expert_begin, expert_end) is stored at the return address recorded for it. */
int qmoe_ep_push_return(const qmoe_route_t* expert_route, uint64_t return_addresses, uint64_t src,
                        const qmoe_ep_peers_t* peers, int32_t expert_begin, int32_t expert_end,
                        int32_t blocks_per_sm, int32_t dtype, int64_t width, uint64_t stream);

/* Barrier over peer memory for the direct transport, without NCCL: every rank writes `sequence`
 * (positive, growing by one per barrier, the same on every rank) into its slot of every rank's flag
 * array (`flags->buffer[p]` = i32 [world] array of rank p, zero at start) and waits, for a bounded time
 * (qmoe_ep_set_barrier_timeout_ms), for all slots of its own array; a rank that never arrives shows up as a non-zero
 * qmoe_device_status on the others, not as a hang.  With stats_local != 0 the kernel first copies this
 * rank's stats_words words into slot `rank` of every rank's table (`stats_tables->buffer[p]` = i32
 * [world, stats_words]): the all-gather of qmoe_ep_gather_stats without NCCL (pack the words first
 * with qmoe_ep_pack_stats). */
int qmoe_ep_flag_barrier(const qmoe_ep_peers_t* flags, int32_t sequence, uint64_t stats_local,
                         int32_t stats_words, const qmoe_ep_peers_t* stats_tables, uint64_t stream);
int qmoe_ep_pack_stats(const qmoe_route_t* route, uint64_t stats_local, uint64_t stream);
/* How long qmoe_ep_flag_barrier waits for the other ranks before it gives up (default 10 000 ms: seconds of
 * skew between the hosts of a training job are normal); applies to barriers enqueued afterwards. */
int qmoe_ep_set_barrier_timeout_ms(int64_t milliseconds);

/* Fused producers (no upstream counterpart): the kernel that creates a row stores it directly in the
 * destination GPU's buffer, so dispatch and combine need no pass of their own.
 *   qmoe_ep_permute_push            x[t] -> the k expert-side rows of token t (peers: every rank's expert-side
 *                                   input buffer and return table); replaces qmoe_permute + qmoe_ep_push_dispatch
 *   qmoe_ep_combine_backward_push   g[t] * w[t, s] -> the expert-side dY rows, d_gate_weights locally (y_local:
 *                                   this rank's combine input); replaces qmoe_combine_backward + push
 *   qmoe_ep_expert_down_push        Y = H Wd^T on the tensor cores, every output row stored at its return
 *   qmoe_ep_expert_dx_push          dX = dG Wg + dU Wu address (peers: every rank's token-side buffer)
 * The two tensor-core variants need bf16 activations and widths that are multiples of 8 (else
 * QMOE_ERR_UNSUPPORTED: use the unfused entry points).  Order a qmoe_ep_barrier after each before the
 * destination is read.
 * The _range forms move only the slots whose expert is one of the owner's local experts [local_begin, local_end)
 * (every rank's experts with those local numbers): a host sends one group of experts, starts the first product on
 * it, and lets the rest travel meanwhile. */
int qmoe_ep_permute_push(const qmoe_route_t* token_route, uint64_t dest_base, uint64_t x,
                         const qmoe_ep_peers_t* peers, int32_t dtype, int64_t width, uint64_t stream);
int qmoe_ep_permute_push_range(const qmoe_route_t* token_route, uint64_t dest_base, uint64_t x,
                               const qmoe_ep_peers_t* peers, int32_t local_begin, int32_t local_end, int32_t dtype,
                               int64_t width, uint64_t stream);
int qmoe_ep_combine_backward_push_range(const qmoe_route_t* token_route, uint64_t dest_base, uint64_t grad_out,
                                        uint64_t y_local, const qmoe_ep_peers_t* peers, uint64_t d_gate_weights,
                                        int32_t local_begin, int32_t local_end, int32_t dtype, int64_t width,
                                        uint64_t stream);
int qmoe_ep_combine_backward_push(const qmoe_route_t* token_route, uint64_t dest_base, uint64_t grad_out,
                                  uint64_t y_local, const qmoe_ep_peers_t* peers, uint64_t d_gate_weights,
                                  int32_t dtype, int64_t width, uint64_t stream);
int qmoe_ep_expert_down_push(const qmoe_route_t* expert_route, const qmoe_experts_t* experts, uint64_t h,
                             uint64_t return_addresses, const qmoe_ep_peers_t* peers, uint64_t stream);
int qmoe_ep_expert_dx_push(const qmoe_route_t* expert_route, const qmoe_experts_t* experts, uint64_t d_g,
                           uint64_t d_u, uint64_t return_addresses, const qmoe_ep_peers_t* peers, uint64_t stream);

/* ---------------------------------------------------------------------------------------------
 * The optimizer step either side of the layer: AdamW and the global gradient-norm clip over many
 * parameter tensors in one launch.  Upstream loops over the parameters and launches one element-wise
 * kernel per tensor for AdamW (src/qutai/nn/optimizers.py:136-153 -> adamw_step_into,
 * src/qutai/backends/cuda.py:449-452, kernel src/qutai/backends/cuda/tensor.cu:101-104) and two
 * reductions plus one scaling per tensor for the clip (src/qutai/nn/optimizers.py:19-31 ->
 * global_norm src/qutai/backends/cuda.py:425-437, scale_into :150-154).
 *
 * The caller lists the tensors that have a gradient (upstream skips `parameter.grad is None`) in a host
 * array of items and passes a device buffer of qmoe_optim_table_bytes(count) bytes the array is copied
 * into; `first_chunk` is filled in by the library.  fp32 parameters, gradients and moments.
 * ------------------------------------------------------------------------------------------- */
typedef struct qmoe_optim_item {
    uint64_t values;      /* [size] fp32 parameter, updated in place */
    uint64_t grad;        /* [size] fp32 gradient */
    uint64_t exp_avg;     /* [size] fp32 first moment, updated in place (zeros before the first step) */
    uint64_t exp_avg_sq;  /* [size] fp32 second moment, updated in place */
    uint64_t shadow;      /* [size] bf16 copy of the updated parameter (the tensor-core operand), or 0 */
    int64_t size;
    int64_t first_chunk;  /* set by the library */
    float c1, c2;         /* bias corrections 1 - beta1^step, 1 - beta2^step of THIS tensor's step count */
} qmoe_optim_item_t;
int64_t qmoe_optim_table_bytes(int32_t count);
/* m = b1 m + (1-b1) g;  v = b2 v + (1-b2) g^2;  p = p (1 - lr wd) - lr (m / c1) / (sqrt(v / c2) + eps), in
 * fp32 in exactly this order (the upstream kernel's); shadow = bf16(p) when given.  `items` may be
 * modified (first_chunk).  Negative settings or betas outside [0, 1) are argument errors, as upstream. */
int qmoe_adamw_multi(qmoe_optim_item_t* items, int32_t count, uint64_t table, float learning_rate, float beta1,
                     float beta2, float eps, float weight_decay, uint64_t stream);
/* L2 norm of all listed gradients (sum of squares in double, fixed order: run-to-run identical) and, when
 * it exceeds max_norm, every gradient scaled by max_norm / norm.  scratch: qmoe_clip_scratch_bytes() bytes;
 * afterwards scratch[0] (double) holds the norm before clipping and scratch[1] the factor applied.  Only
 * `grad` and `size` of the items are read.  Upstream raises for a non-finite norm after reading it back;
 * here a non-finite norm leaves the gradients unscaled and the host decides when it reads scratch[0]. */
int64_t qmoe_clip_scratch_bytes(void);
int qmoe_clip_grad_norm(qmoe_optim_item_t* items, int32_t count, uint64_t table, double max_norm, uint64_t scratch,
                        uint64_t stream);

#ifdef __cplusplus
}
#endif
#endif /* QUTAI_MOE_H */
