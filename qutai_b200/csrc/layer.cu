// Expert FFN forward/backward (engine selection between the tcgen05 kernels and the CUDA-core
// kernels), the single-group GEMM of the host function table, and the whole-layer entry points.
#include <atomic>

#include "common.cuh"

namespace qmoe {

namespace {

int check_experts(const qmoe_route_t* r, const qmoe_experts_t* ex, int* engine) {
    if (int rc = route_check(r)) return rc;
    if (!ex) return fail_arg("experts is null");
    if (ex->experts != r->experts) return fail_arg("experts.experts (%d) differs from route.experts (%d)", ex->experts, r->experts);
    if (ex->dtype != QMOE_F32 && ex->dtype != QMOE_BF16) return fail_arg("experts.dtype must be QMOE_F32 or QMOE_BF16");
    if (ex->width <= 0 || ex->hidden <= 0) return fail_arg("experts.width and experts.hidden must be positive");
    if (!ex->w_gate || !ex->w_up || !ex->w_down) return fail_arg("experts has a null weight address");
    int e = ex->engine;
    const bool tc_ok = ex->dtype == QMOE_BF16 && tcgen05_shape_ok(ex->width, ex->hidden);
    if (e == QMOE_ENGINE_AUTO) e = tc_ok ? QMOE_ENGINE_TCGEN05 : QMOE_ENGINE_SIMT;
    if (e == QMOE_ENGINE_TCGEN05 && !tc_ok) {
        set_error("the tcgen05 engine needs bf16 activations and widths that are multiples of 8 (d %lld, h %lld, dtype %d)",
                  (long long)ex->width, (long long)ex->hidden, ex->dtype);
        return QMOE_ERR_UNSUPPORTED;
    }
    if (e != QMOE_ENGINE_TCGEN05 && e != QMOE_ENGINE_SIMT) return fail_arg("experts.engine %d is unknown", ex->engine);
    *engine = e;
    return 0;
}

// C[rows, N] = A[rows, K] . op(B_e) on CUDA cores; b_kfast: B_e is [N, K] ("x W^T"), else [K, N]
int simt_rows(const qmoe_route_t* r, const qmoe_experts_t* ex, uint64_t a, uint64_t b, uint64_t a2, uint64_t b2, uint64_t c,
              long long K, long long N, bool b_kfast, cudaStream_t stream) {
    SimtGemmArgs g = {};
    g.A = (const void*)a; g.B = (const void*)b; g.A2 = (const void*)a2; g.B2 = (const void*)b2; g.C = (void*)c;
    g.M = r->rows_bound; g.N = N; g.K = K;
    g.a_rs = K; g.a_cs = 1;
    g.b_rs = b_kfast ? 1 : N; g.b_cs = b_kfast ? K : 1;
    g.ldc = N; g.mode = SG_ROWS;
    g.tile_expert = (const int*)r->tile_expert; g.meta = (const int*)r->meta;
    g.b_slab = K * N;
    return launch_simt_gemm(g, ex->dtype, ex->dtype, ex->dtype, r->rows_bound, 1, stream);
}

// C_e[M, N] (fp32) = A_e^T . B_e, A [rows, M], B [rows, N]
int simt_wgrad(const qmoe_route_t* r, const qmoe_experts_t* ex, uint64_t a, uint64_t b, uint64_t c, long long M, long long N,
               cudaStream_t stream) {
    SimtGemmArgs g = {};
    g.A = (const void*)a; g.B = (const void*)b; g.C = (void*)c;
    g.M = M; g.N = N; g.K = 0;
    g.a_rs = 1; g.a_cs = M;
    g.b_rs = N; g.b_cs = 1;
    g.ldc = N; g.mode = SG_K;
    g.offsets = (const int*)r->offsets; g.counts = (const int*)r->counts;
    g.c_slab = M * N;
    return launch_simt_gemm(g, ex->dtype, ex->dtype, QMOE_F32, M, ex->experts, stream);
}

}  // namespace
}  // namespace qmoe

using namespace qmoe;

extern "C" int qmoe_expert_forward_parts(const qmoe_route_t* r, const qmoe_experts_t* ex, uint64_t x, uint64_t g, uint64_t u,
                                         uint64_t h, uint64_t y, int32_t parts, uint64_t stream_) {
    int engine = 0;
    if (int rc = check_experts(r, ex, &engine)) return rc;
    if (!(parts & (QMOE_FWD_UP | QMOE_FWD_DOWN)) || (parts & ~(QMOE_FWD_UP | QMOE_FWD_DOWN)))
        return fail_arg("expert_forward: parts must be a combination of QMOE_FWD_UP and QMOE_FWD_DOWN");
    if (!h || ((parts & QMOE_FWD_UP) && (!x || !g || !u)) || ((parts & QMOE_FWD_DOWN) && !y))
        return fail_arg("expert_forward: null buffer address");
    cudaStream_t stream = (cudaStream_t)stream_;
    const long long d = ex->width, hd = ex->hidden;
    const bool tc = engine == QMOE_ENGINE_TCGEN05;
    if (parts & QMOE_FWD_UP) {
        if (tc) {
            TimedScope timed(KC_EXPERT_GEMM, stream);
            if (int rc = tc_swiglu_forward(r, ex, x, g, u, h, stream)) return rc;
        } else {
            {
                TimedScope timed(KC_EXPERT_GEMM, stream);
                if (int rc = simt_rows(r, ex, x, ex->w_gate, 0, 0, g, d, hd, true, stream)) return rc;
                if (int rc = simt_rows(r, ex, x, ex->w_up, 0, 0, u, d, hd, true, stream)) return rc;
            }
            if (int rc = launch_swiglu(r, g, u, h, ex->dtype, hd, stream)) return rc;
        }
    }
    if (parts & QMOE_FWD_DOWN) {
        TimedScope timed(KC_EXPERT_GEMM, stream);
        return tc ? tc_rows_nt(r, ex->experts, h, ex->w_down, y, hd, d, stream)
                  : simt_rows(r, ex, h, ex->w_down, 0, 0, y, hd, d, true, stream);
    }
    return 0;
}

extern "C" int qmoe_expert_forward(const qmoe_route_t* r, const qmoe_experts_t* ex, uint64_t x, uint64_t g, uint64_t u,
                                   uint64_t h, uint64_t y, uint64_t stream) {
    return qmoe_expert_forward_parts(r, ex, x, g, u, h, y, QMOE_FWD_UP | QMOE_FWD_DOWN, stream);
}

extern "C" int qmoe_expert_backward_parts(const qmoe_route_t* r, const qmoe_experts_t* ex, uint64_t dy, uint64_t x, uint64_t g,
                                          uint64_t u, uint64_t h, uint64_t d_h, uint64_t d_g, uint64_t d_u, uint64_t dx,
                                          uint64_t d_w_gate, uint64_t d_w_up, uint64_t d_w_down, int32_t parts,
                                          uint64_t stream_) {
    int engine = 0;
    if (int rc = check_experts(r, ex, &engine)) return rc;
    const bool skip_dx = (parts & QMOE_BWD_NO_DX) != 0;
    parts &= ~QMOE_BWD_NO_DX;
    if (!(parts & (QMOE_BWD_ACTIVATIONS | QMOE_BWD_WEIGHTS)) || (parts & ~(QMOE_BWD_ACTIVATIONS | QMOE_BWD_WEIGHTS)))
        return fail_arg("expert_backward: parts must be a combination of QMOE_BWD_ACTIVATIONS and QMOE_BWD_WEIGHTS");
    if (!dy || !x || !g || !u || !h || !d_h || !d_g || !d_u) return fail_arg("expert_backward: null buffer address");
    if ((parts & QMOE_BWD_ACTIVATIONS) && !skip_dx && !dx) return fail_arg("expert_backward: dx is null");
    if ((parts & QMOE_BWD_WEIGHTS) && (!d_w_gate || !d_w_up || !d_w_down)) return fail_arg("expert_backward: null gradient address");
    if (parts == QMOE_BWD_ACTIVATIONS && !skip_dx && dx == dy)
        return fail_arg("expert_backward: dx may alias dy only when both parts run in one call");
    cudaStream_t stream = (cudaStream_t)stream_;
    const long long d = ex->width, hd = ex->hidden;
    const bool tc = engine == QMOE_ENGINE_TCGEN05;
    if (parts & QMOE_BWD_ACTIVATIONS) {
        if (tc) {  // dG, dU straight from the accumulator of dH = dY . Wd (dH itself is never stored)
            TimedScope timed(KC_EXPERT_GEMM, stream);
            if (int rc = tc_dswiglu(r, ex->experts, dy, ex->w_down, g, u, d_g, d_u, d, hd, stream)) return rc;
        } else {
            {
                TimedScope timed(KC_EXPERT_GEMM, stream);
                if (int rc = simt_rows(r, ex, dy, ex->w_down, 0, 0, d_h, d, hd, false, stream)) return rc;
            }
            if (int rc = launch_swiglu_backward(r, d_h, g, u, d_g, d_u, ex->dtype, hd, stream)) return rc;
        }
        if (!skip_dx && dx != dy) {  // dX first when it has a buffer of its own: a host can ship it while the weight gradients run
            TimedScope timed(KC_EXPERT_GEMM, stream);
            if (int rc = tc ? tc_rows_nn(r, ex->experts, d_g, ex->w_gate, d_u, ex->w_up, dx, hd, d, stream)
                            : simt_rows(r, ex, d_g, ex->w_gate, d_u, ex->w_up, dx, hd, d, false, stream)) return rc;
        }
    }
    if (parts & QMOE_BWD_WEIGHTS) {
        TimedScope timed(KC_WGRAD_GEMM, stream);
        if (tc) {  // all three in one launch
            if (int rc = tc_wgrad3(r, ex->experts, dy, h, x, d_g, d_u, d_w_down, d_w_gate, d_w_up, d, hd, stream)) return rc;
        } else {
            if (int rc = simt_wgrad(r, ex, dy, h, d_w_down, d, hd, stream)) return rc;
            if (int rc = simt_wgrad(r, ex, d_g, x, d_w_gate, hd, d, stream)) return rc;
            if (int rc = simt_wgrad(r, ex, d_u, x, d_w_up, hd, d, stream)) return rc;
        }
    }
    if ((parts & QMOE_BWD_ACTIVATIONS) && !skip_dx && dx == dy) {  // dX overwrites dY: only after dY's last reader (dWd)
        TimedScope timed(KC_EXPERT_GEMM, stream);
        return tc ? tc_rows_nn(r, ex->experts, d_g, ex->w_gate, d_u, ex->w_up, dx, hd, d, stream)
                  : simt_rows(r, ex, d_g, ex->w_gate, d_u, ex->w_up, dx, hd, d, false, stream);
    }
    return 0;
}

extern "C" int qmoe_expert_backward(const qmoe_route_t* r, const qmoe_experts_t* ex, uint64_t dy, uint64_t x, uint64_t g,
                                    uint64_t u, uint64_t h, uint64_t d_h, uint64_t d_g, uint64_t d_u, uint64_t dx,
                                    uint64_t d_w_gate, uint64_t d_w_up, uint64_t d_w_down, uint64_t stream) {
    return qmoe_expert_backward_parts(r, ex, dy, x, g, u, h, d_h, d_g, d_u, dx, d_w_gate, d_w_up, d_w_down,
                                      QMOE_BWD_ACTIVATIONS | QMOE_BWD_WEIGHTS, stream);
}

// ---- plain products on the tensor cores: the grouped kernels with ONE group --------------------------------------
namespace qmoe {
namespace {
constexpr int kGroupSlots = 256;                 // products in flight at once that may each need a table of their own
__device__ int g_group_tables[kGroupSlots * 4];  // per slot: offsets {0, rows}, counts {rows}
__global__ void fill_group_kernel(int* table, int rows) { table[0] = 0; table[1] = rows; table[2] = rows; table[3] = 0; }

// the one-group route of a product with `rows` rows (nullptr and an error recorded when the table cannot be reached)
int one_group_route(qmoe_route_t* r, long long rows, cudaStream_t stream) {
    static std::atomic<unsigned> next{0};
    static int* base[64] = {nullptr};
    int dev = 0;
    QMOE_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= 64) return fail_arg("gemm: device index out of range");
    if (!base[dev]) {
        void* address = nullptr;
        QMOE_CUDA(cudaGetSymbolAddress(&address, g_group_tables));
        base[dev] = (int*)address;
    }
    int* table = base[dev] + 4 * (next.fetch_add(1, std::memory_order_relaxed) % kGroupSlots);
    fill_group_kernel<<<1, 1, 0, stream>>>(table, (int)rows);
    QMOE_LAUNCH_CHECK("fill_group_kernel");
    *r = qmoe_route_t{};
    r->rows_bound = rows;
    r->offsets = (uint64_t)table;
    r->counts = (uint64_t)(table + 2);
    return 0;
}
}  // namespace
}  // namespace qmoe

// Plain product.  bf16 x bf16 in the three forms a linear layer needs goes to the tcgen05 kernels (A [M, K] . B[N, K]^T and
// A [M, K] . B [K, N] with bf16 results and M a multiple of 128, the rows a tile writes; A [K, M]^T . B [K, N] with fp32
// results: a weight gradient); everything else, and every accumulating call, to the CUDA-core kernel.
extern "C" int qmoe_gemm(uint64_t a, int32_t a_dtype, uint64_t b, int32_t b_dtype, uint64_t c, int32_t c_dtype, int64_t m,
                         int64_t k, int64_t n, int32_t transpose_a, int32_t transpose_b, int32_t accumulate, uint64_t stream_) {
    if (!a || !b || !c) return fail_arg("gemm: null address");
    if (m <= 0 || n <= 0 || k <= 0) return fail_arg("gemm: sizes must be positive");
    for (int dt : {a_dtype, b_dtype, c_dtype})
        if (dt != QMOE_F32 && dt != QMOE_BF16) return fail_arg("gemm: dtype must be QMOE_F32 or QMOE_BF16");
    if (c == a || c == b) return fail_arg("gemm: the output must not alias an input");
    cudaStream_t stream = (cudaStream_t)stream_;
    const bool aligned = !((a | b | c) & 15u) && k % 8 == 0 && n % 8 == 0 && m % 8 == 0 && m < (1ll << 30) && k < (1ll << 30) && n < (1ll << 30);
    if (a_dtype == QMOE_BF16 && b_dtype == QMOE_BF16 && aligned && !accumulate && !kernel_variant(QMOE_VARIANT_PLAIN_GEMM_ON_CUDA_CORES)) {
        qmoe_route_t r;
        if (!transpose_a && c_dtype == QMOE_BF16 && m % kRowPad == 0) {
            TimedScope timed(KC_EXPERT_GEMM, stream);
            if (int rc = one_group_route(&r, m, stream)) return rc;
            return transpose_b ? tc_rows_nt(&r, 1, a, b, c, k, n, stream, nullptr) : tc_rows_nn(&r, 1, a, b, 0, 0, c, k, n, stream, nullptr);
        }
        if (transpose_a && !transpose_b && c_dtype == QMOE_F32) {
            TimedScope timed(KC_WGRAD_GEMM, stream);
            if (int rc = one_group_route(&r, k, stream)) return rc;     // the contraction runs over the k rows of both operands
            return tc_wgrad1(&r, a, b, c, m, n, stream);
        }
    }
    TimedScope timed(KC_OTHER, stream);
    SimtGemmArgs g = {};
    g.A = (const void*)a; g.B = (const void*)b; g.C = (void*)c;
    g.M = m; g.N = n; g.K = k;
    g.a_rs = transpose_a ? 1 : k; g.a_cs = transpose_a ? m : 1;
    g.b_rs = transpose_b ? 1 : n; g.b_cs = transpose_b ? k : 1;
    g.ldc = n; g.accumulate = accumulate; g.mode = SG_PLAIN;
    return launch_simt_gemm(g, a_dtype, b_dtype, c_dtype, m, 1, stream);
}

// ---- the weight gradient of a linear layer, its rows cut into ranges that run side by side ---------------------------
namespace qmoe {
namespace {
constexpr int kSplitTableInts = 64;      // at the head of the scratch: offsets[splits + 1], counts[splits]
constexpr int kMaxSplits = 16;

long long split_rows(long long k, int splits) { return ((k + splits - 1) / splits + kRowPad - 1) / kRowPad * kRowPad; }
// how many row ranges make m x n tiles of 256 x 256 fill the CTA pairs once, each range at least 512 rows long
int wgrad_splits(long long m, long long k, long long n) {
    const long long tiles = ((m + 255) / 256) * ((n + 255) / 256), pairs = sm_count() / 2;
    long long splits = pairs / tiles;
    if (splits > k / 512) splits = k / 512;
    if (splits > kMaxSplits) splits = kMaxSplits;
    if (splits < 2) return 1;
    const long long rows = split_rows(k, (int)splits);
    return (int)((k + rows - 1) / rows);        // ranges start on multiples of 128 rows: none of them may come out empty
}

__global__ void fill_split_table_kernel(int* table, int splits, int rows_per_split, int rows) {
    const int i = threadIdx.x;
    if (i <= splits) table[i] = i * rows_per_split;
    if (i < splits) {
        const int left = rows - i * rows_per_split;
        table[splits + 1 + i] = left < 0 ? 0 : (left > rows_per_split ? rows_per_split : left);
    }
}
// out = slab 0 + slab 1 + ... in that order, four values per thread
__global__ void __launch_bounds__(256) sum_slabs_kernel(const float4* __restrict__ slabs, float4* __restrict__ out, int count, long long quads) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < quads; i += (long long)gridDim.x * blockDim.x) {
        float4 total = slabs[i];
        for (int s = 1; s < count; ++s) {
            const float4 v = slabs[(long long)s * quads + i];
            total.x += v.x; total.y += v.y; total.z += v.z; total.w += v.w;
        }
        out[i] = total;
    }
}
}  // namespace
}  // namespace qmoe

extern "C" int64_t qmoe_gemm_wgrad_partials(int64_t m, int64_t k, int64_t n) {
    if (m <= 0 || k <= 0 || n <= 0 || m % 8 || n % 8 || k % 8) return 0;
    const int splits = wgrad_splits(m, k, n);
    return splits < 2 ? 0 : kSplitTableInts + (int64_t)splits * m * n;
}

extern "C" int qmoe_gemm_wgrad_split(uint64_t a, uint64_t b, uint64_t c, uint64_t partials, int64_t m, int64_t k, int64_t n,
                                     uint64_t stream_) {
    if (!a || !b || !c || !partials) return fail_arg("gemm_wgrad_split: null address");
    if ((a | b | c | partials) & 15u) return fail_arg("gemm_wgrad_split: addresses must be multiples of 16 bytes");
    if (c == a || c == b) return fail_arg("gemm_wgrad_split: the output must not alias an input");
    if (m <= 0 || k <= 0 || n <= 0 || m % 8 || n % 8 || k % 8 || k >= (1ll << 30)) return fail_arg("gemm_wgrad_split: sizes must be positive multiples of 8");
    const int splits = wgrad_splits(m, k, n);
    if (splits < 2) return fail_arg("gemm_wgrad_split: this shape is not split (qmoe_gemm_wgrad_partials gives 0): use qmoe_gemm");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_WGRAD_GEMM, stream);
    int* table = (int*)partials;
    float* slabs = (float*)partials + kSplitTableInts;
    fill_split_table_kernel<<<1, 32, 0, stream>>>(table, splits, (int)split_rows(k, splits), (int)k);
    QMOE_LAUNCH_CHECK("fill_split_table_kernel");
    qmoe_route_t r = {};
    r.rows_bound = k;
    r.offsets = (uint64_t)table;
    r.counts = (uint64_t)(table + splits + 1);
    if (int rc = tc_wgrad1(&r, a, b, (uint64_t)slabs, m, n, stream, splits, m * n)) return rc;
    const long long quads = m * n / 4;
    long long blocks = (quads + 255) / 256;
    if (blocks > 8ll * sm_count()) blocks = 8ll * sm_count();
    sum_slabs_kernel<<<(unsigned)blocks, 256, 0, stream>>>((const float4*)slabs, (float4*)c, splits, quads);
    QMOE_LAUNCH_CHECK("sum_slabs_kernel");
    return 0;
}

extern "C" int qmoe_layer_forward(const qmoe_layer_t* L, uint64_t stream) {
    if (!L) return fail_arg("layer is null");
    const qmoe_route_t* r = &L->route;
    const qmoe_experts_t* ex = &L->experts;
    int engine = 0;
    if (int rc = check_experts(r, ex, &engine)) return rc;
    if (!L->x || !L->w_router || !L->scores || !L->x_dispatched || !L->g || !L->u || !L->h || !L->y_dispatched || !L->out)
        return fail_arg("layer_forward: null buffer address");
    const long long d = ex->width, hd = ex->hidden, E = ex->experts;
    if (ex->dtype == QMOE_BF16 && L->master_gate) {
        if (!L->master_up || !L->master_down) return fail_arg("layer_forward: master weights must be given together");
        if (int rc = qmoe_cast_bf16(L->master_gate, ex->w_gate, E * hd * d, stream)) return rc;
        if (int rc = qmoe_cast_bf16(L->master_up, ex->w_up, E * hd * d, stream)) return rc;
        if (int rc = qmoe_cast_bf16(L->master_down, ex->w_down, E * hd * d, stream)) return rc;
    }
    if (int rc = qmoe_router_forward(L->x, ex->dtype, L->w_router, L->scores, L->router_partials, r->tokens, d, r->experts, stream)) return rc;
    if (int rc = qmoe_route(r, L->scores, stream)) return rc;
    if (int rc = qmoe_permute(r, L->x, L->x_dispatched, ex->dtype, d, stream)) return rc;
    if (int rc = qmoe_expert_forward(r, ex, L->x_dispatched, L->g, L->u, L->h, L->y_dispatched, stream)) return rc;
    return qmoe_combine(r, L->y_dispatched, L->out, ex->dtype, d, stream);
}

extern "C" int qmoe_layer_backward(const qmoe_layer_t* L, uint64_t stream) {
    if (!L) return fail_arg("layer is null");
    const qmoe_route_t* r = &L->route;
    const qmoe_experts_t* ex = &L->experts;
    int engine = 0;
    if (int rc = check_experts(r, ex, &engine)) return rc;
    if (!L->grad_out || !L->dy_dispatched || !L->d_h || !L->d_g || !L->d_u || !L->dx_dispatched || !L->d_gate_weights ||
        !L->d_scores || !L->dx_router || !L->router_partials || !L->dx || !L->d_w_router)
        return fail_arg("layer_backward: null buffer address");
    const long long d = ex->width;
    if (int rc = qmoe_combine_backward(r, L->grad_out, L->y_dispatched, L->dy_dispatched, L->d_gate_weights, ex->dtype, d, stream)) return rc;
    if (int rc = qmoe_expert_backward(r, ex, L->dy_dispatched, L->x_dispatched, L->g, L->u, L->h, L->d_h, L->d_g, L->d_u,
                                      L->dx_dispatched, L->d_w_gate, L->d_w_up, L->d_w_down, stream)) return rc;
    if (int rc = qmoe_route_backward(r, L->d_gate_weights, L->grad_aux, L->d_scores, stream)) return rc;
    if (int rc = qmoe_router_backward(L->d_scores, L->x, ex->dtype, L->w_router, L->dx_router, L->d_w_router,
                                      L->router_partials, r->tokens, d, r->experts, stream)) return rc;
    return qmoe_unpermute_reduce(r, L->dx_dispatched, L->dx_router, L->dx, ex->dtype, d, stream);
}

// ---- the block's feed-forward half with the norm and the residual fused in -------------------------------
namespace {
int check_block(const qmoe_block_t* B) {
    if (!B) return fail_arg("block is null");
    if (!B->norm_weight || !B->inverse || !B->w_router_folded) return fail_arg("block: null norm weight / inverse / folded router address");
    if (!(B->norm_eps >= 0)) return fail_arg("block: norm_eps must not be negative");
    return 0;
}
}  // namespace

extern "C" int qmoe_block_forward(const qmoe_block_t* B, uint64_t stream) {
    if (int rc = check_block(B)) return rc;
    const qmoe_layer_t* L = &B->layer;
    const qmoe_route_t* r = &L->route;
    const qmoe_experts_t* ex = &L->experts;
    int engine = 0;
    if (int rc = check_experts(r, ex, &engine)) return rc;
    if (!L->x || !L->w_router || !L->scores || !L->x_dispatched || !L->g || !L->u || !L->h || !L->y_dispatched || !L->out)
        return fail_arg("block_forward: null buffer address");
    if (L->out == L->x) return fail_arg("block_forward: the output must not alias the input (the backward re-reads it)");
    const long long d = ex->width, hd = ex->hidden, E = ex->experts;
    if (ex->dtype == QMOE_BF16 && L->master_gate) {
        if (!L->master_up || !L->master_down) return fail_arg("block_forward: master weights must be given together");
        if (int rc = qmoe_cast_bf16(L->master_gate, ex->w_gate, E * hd * d, stream)) return rc;
        if (int rc = qmoe_cast_bf16(L->master_up, ex->w_up, E * hd * d, stream)) return rc;
        if (int rc = qmoe_cast_bf16(L->master_down, ex->w_down, E * hd * d, stream)) return rc;
    }
    // scores = rms_norm(x) . W_r^T = inverse[t] * (x . (W_r * w)^T): the product reads the raw activations
    if (int rc = qmoe_rms_inverse(L->x, ex->dtype, B->inverse, r->tokens, d, B->norm_eps, stream)) return rc;
    if (int rc = qmoe_scale_f32(L->w_router, B->w_router_folded, 0, B->norm_weight, E, d, stream)) return rc;
    if (int rc = qmoe_router_forward(L->x, ex->dtype, B->w_router_folded, L->scores, L->router_partials, r->tokens, d, r->experts, stream)) return rc;
    if (int rc = qmoe_scale_f32(L->scores, L->scores, B->inverse, 0, r->tokens, E, stream)) return rc;
    if (int rc = qmoe_route(r, L->scores, stream)) return rc;
    if (int rc = qmoe_permute_norm(r, L->x, B->inverse, B->norm_weight, L->x_dispatched, ex->dtype, d, stream)) return rc;
    if (int rc = qmoe_expert_forward(r, ex, L->x_dispatched, L->g, L->u, L->h, L->y_dispatched, stream)) return rc;
    return qmoe_combine_residual(r, L->y_dispatched, L->x, L->out, ex->dtype, d, stream);
}

extern "C" int qmoe_block_backward(const qmoe_block_t* B, uint64_t stream) {
    if (int rc = check_block(B)) return rc;
    const qmoe_layer_t* L = &B->layer;
    const qmoe_route_t* r = &L->route;
    const qmoe_experts_t* ex = &L->experts;
    int engine = 0;
    if (int rc = check_experts(r, ex, &engine)) return rc;
    if (!L->grad_out || !L->dy_dispatched || !L->d_h || !L->d_g || !L->d_u || !L->dx_dispatched || !L->d_gate_weights ||
        !L->d_scores || !L->dx_router || !L->router_partials || !L->dx || !L->d_w_router || !B->d_norm_weight ||
        !B->norm_partials)
        return fail_arg("block_backward: null buffer address");
    const long long d = ex->width, E = ex->experts;
    if (int rc = qmoe_combine_backward(r, L->grad_out, L->y_dispatched, L->dy_dispatched, L->d_gate_weights, ex->dtype, d, stream)) return rc;
    if (int rc = qmoe_expert_backward(r, ex, L->dy_dispatched, L->x_dispatched, L->g, L->u, L->h, L->d_h, L->d_g, L->d_u,
                                      L->dx_dispatched, L->d_w_gate, L->d_w_up, L->d_w_down, stream)) return rc;
    if (int rc = qmoe_route_backward(r, L->d_gate_weights, L->grad_aux, L->d_scores, stream)) return rc;
    // router: the weight gradient is d_scores^T . rms_norm(x) = ((inverse * d_scores)^T . x) * w, from the raw
    // activations; the same product call returns (inverse * d_scores) . W_r, i.e. inverse[t] times the gradient of
    // the NORMALISED input, and the kernel below takes the row scale back out
    if (int rc = qmoe_scale_f32(L->d_scores, L->d_scores, B->inverse, 0, r->tokens, E, stream)) return rc;
    if (int rc = qmoe_router_backward(L->d_scores, L->x, ex->dtype, L->w_router, L->dx_router, L->d_w_router, L->router_partials,
                                      r->tokens, d, r->experts, stream)) return rc;
    if (int rc = qmoe_scale_f32(L->d_w_router, L->d_w_router, 0, B->norm_weight, E, d, stream)) return rc;
    return qmoe_unpermute_norm_backward(r, L->dx_dispatched, L->dx_router, 1, L->x, B->inverse, B->norm_weight, L->grad_out,
                                        L->dx, B->d_norm_weight, B->norm_partials, ex->dtype, d, stream);
}
