// Routing: softmax / top-k gating, per-expert counts, padded offsets, stable dispatch permutation,
// utilisation, auxiliary loss and the routing backward.  All tables are produced on the device
// with no host synchronisation and no floating-point atomics (results are run-to-run identical).
//
// Semantics follow `routing` / `routing_backward` of the upstream CPU path
// (src/qutai/backends/cpu_lm.py:204-276): experts are ranked by probability, equal values keep the
// lower expert index first, the k selected probabilities are renormalised to sum to one, and inside
// one expert the routed rows keep increasing (token, slot) order.
#include <limits.h>

#include "common.cuh"

namespace qmoe {

namespace {

constexpr int kWarps = 8;
constexpr int kRowsPerWarp = kRouteRowsPerBlock / kWarps;  // 4

// ---- K1: softmax + top-k + per-block histogram and probability column sums --------------------
// One warp per token row; lane l holds experts l, l+32, ... (EPL of them).  Ranking uses the raw
// scores: softmax is strictly monotone, so this is the ranking by exact probability, without the
// extra ties that rounding the probabilities to fp32 would create.
template <int EPL>
__global__ void __launch_bounds__(kWarps * 32)
route_topk_kernel(const float* __restrict__ scores, float* __restrict__ probs,
                  float* __restrict__ gate_w, int* __restrict__ expert_idx,
                  int* __restrict__ block_counts, float* __restrict__ block_colsum,
                  long long T, int E, int k) {
    __shared__ int s_cnt[kMaxExperts];
    __shared__ float s_col[kWarps][kMaxExperts];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < E; i += blockDim.x) s_cnt[i] = 0;
    __syncthreads();

    float col[EPL];
#pragma unroll
    for (int j = 0; j < EPL; ++j) col[j] = 0.f;

    const long long row0 = (long long)blockIdx.x * kRouteRowsPerBlock + warp * kRowsPerWarp;
    for (int r = 0; r < kRowsPerWarp; ++r) {
        const long long row = row0 + r;
        if (row >= T) break;
        float v[EPL], p[EPL];
        float m = -INFINITY;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            const int e = lane + 32 * j;
            v[j] = e < E ? scores[row * E + e] : -INFINITY;
            m = fmaxf(m, v[j]);
        }
        m = warp_max(m);
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            const int e = lane + 32 * j;
            p[j] = e < E ? expf(v[j] - m) : 0.f;
            s += p[j];
        }
        s = warp_sum(s);
#pragma unroll
        for (int j = 0; j < EPL; ++j) {
            const int e = lane + 32 * j;
            p[j] = p[j] / s;
            if (e < E) probs[row * E + e] = p[j];
            col[j] += p[j];
        }
        // top-k by (score descending, expert index ascending).  A NaN score ranks as -inf: every comparison below
        // then has the same outcome in every lane, so the lanes agree on each winner (with NaNs left in, each lane
        // would keep its own candidate, mark only that one as taken, and run out of candidates before slot k).
        // The probabilities and gate weights still carry the NaN to the output.
#pragma unroll
        for (int j = 0; j < EPL; ++j)
            if (v[j] != v[j]) v[j] = -INFINITY;
        unsigned taken = 0;
        float wsel[kMaxTopK];
        float total = 0.f;
#pragma unroll
        for (int slot = 0; slot < kMaxTopK; ++slot) {
            wsel[slot] = 0.f;
            if (slot < k) {
                float bv = -INFINITY;
                int be = INT_MAX;
#pragma unroll
                for (int j = 0; j < EPL; ++j) {
                    const int e = lane + 32 * j;
                    if (e < E && !((taken >> j) & 1u) && (be == INT_MAX || v[j] > bv)) {
                        bv = v[j];
                        be = e;
                    }
                }
#pragma unroll
                for (int o = 16; o; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                    const int oe = __shfl_xor_sync(0xffffffffu, be, o);
                    if (oe != INT_MAX && (be == INT_MAX || ov > bv || (ov == bv && oe < be))) {
                        bv = ov;
                        be = oe;
                    }
                }
                float mine = 0.f;
#pragma unroll
                for (int j = 0; j < EPL; ++j)
                    if (j == (be >> 5)) mine = p[j];
                if ((be & 31) == lane) taken |= 1u << (be >> 5);
                const float pw = __shfl_sync(0xffffffffu, mine, be & 31);
                wsel[slot] = pw;
                total += pw;  // left-to-right sum over the slots, like the upstream `sum(...)`
                if (lane == 0) {   // be < E here: k <= E and the ranking is a total order
                    expert_idx[row * k + slot] = be;
                    atomicAdd(&s_cnt[be], 1);  // integer: order does not matter
                }
            }
        }
#pragma unroll
        for (int slot = 0; slot < kMaxTopK; ++slot)
            if (slot < k && lane == slot) gate_w[row * k + slot] = wsel[slot] / total;
    }
#pragma unroll
    for (int j = 0; j < EPL; ++j) {
        const int e = lane + 32 * j;
        if (e < E) s_col[warp][e] = col[j];
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        float t = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) t += s_col[w][e];  // fixed order
        block_colsum[(long long)blockIdx.x * E + e] = t;
        block_counts[(long long)blockIdx.x * E + e] = s_cnt[e];
    }
}

// ---- K2: scan over blocks, padded offsets, tile map, utilisation and auxiliary loss -----------
// One block of 1024 threads: thread (segment, expert) first totals its segment of token blocks, the
// segments are prefixed per expert, then each thread writes the running bases of its segment.  All
// sums run in a fixed order (column sums in double), so the results are run-to-run identical.
constexpr int kScanThreads = 1024;
__global__ void __launch_bounds__(kScanThreads)
route_scan_kernel(const int* __restrict__ block_counts, const float* __restrict__ block_colsum,
                  int* __restrict__ block_base, int* __restrict__ counts, int* __restrict__ offsets,
                  int* __restrict__ tile_expert, int* __restrict__ meta, float* __restrict__ util,
                  float* __restrict__ aux, int nblk, long long T, int E, int k) {
    __shared__ int s_seg[kScanThreads];
    __shared__ double s_segcs[kScanThreads];
    __shared__ int s_cnt[kMaxExperts];
    __shared__ int s_off[kMaxExperts + 1];
    __shared__ double s_cs[kMaxExperts];
    const int nseg = kScanThreads / E;
    const int seg = threadIdx.x / E, e = threadIdx.x - seg * E;
    const bool active = seg < nseg;
    const int chunk = (nblk + nseg - 1) / nseg;
    const int b0 = seg * chunk, b1 = min(nblk, b0 + chunk);
    if (active) {
        int total = 0;
        double cs = 0.0;
        for (int b = b0; b < b1; ++b) {
            total += block_counts[(long long)b * E + e];
            cs += (double)block_colsum[(long long)b * E + e];
        }
        s_seg[threadIdx.x] = total;
        s_segcs[threadIdx.x] = cs;
    }
    __syncthreads();
    if (active) {
        int run = 0;
        for (int s = 0; s < seg; ++s) run += s_seg[s * E + e];
        for (int b = b0; b < b1; ++b) {
            const int c = block_counts[(long long)b * E + e];
            block_base[(long long)b * E + e] = run;
            run += c;
        }
        if (seg == 0) {
            int total = 0;
            double cs = 0.0;
            for (int s = 0; s < nseg; ++s) { total += s_seg[s * E + e]; cs += s_segcs[s * E + e]; }
            counts[e] = total;
            s_cnt[e] = total;
            s_cs[e] = cs;
        }
    }
    __syncthreads();
    const double A = (double)T * k;
    if (threadIdx.x == 0) {
        int off = 0;
        double total = 0.0;
        for (int i = 0; i < E; ++i) {
            s_off[i] = off;
            offsets[i] = off;
            off += (s_cnt[i] + kRowPad - 1) / kRowPad * kRowPad;
            total += ((double)s_cnt[i] / A) * s_cs[i] / (double)T;
        }
        s_off[E] = off;
        offsets[E] = off;
        meta[0] = off;
        meta[1] = off / kRowPad;
        meta[2] = (int)(T * k);
        meta[3] = 0;
        aux[0] = (float)((double)E * total);
    }
    __syncthreads();
    if (threadIdx.x < E) {
        const int x = threadIdx.x;
        util[x] = (float)((double)s_cnt[x] / A);
        for (int t = s_off[x] / kRowPad; t < s_off[x + 1] / kRowPad; ++t) tile_expert[t] = x;
    }
}

// ---- K3: stable rank of every assignment inside (block, expert) -> dispatch tables -----------
// Same block partition as K1.  Warp w owns a contiguous slice of the block's assignments; a
// `match_any` per 32-assignment chunk ranks equal experts by lane, so order is (token, slot).
__global__ void __launch_bounds__(kWarps * 32)
route_pack_kernel(const int* __restrict__ expert_idx, const int* __restrict__ block_base,
                  const int* __restrict__ offsets, int* __restrict__ dest_row,
                  int* __restrict__ row_source, long long T, int E, int k) {
    __shared__ int s_hist[kWarps][kMaxExperts];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int i = threadIdx.x; i < kWarps * kMaxExperts; i += blockDim.x) (&s_hist[0][0])[i] = 0;
    __syncthreads();
    const long long A = T * k;
    const long long begin = ((long long)blockIdx.x * kRouteRowsPerBlock + warp * kRowsPerWarp) * k;
    long long end = begin + (long long)kRowsPerWarp * k;
    if (end > A) end = A;
    const unsigned lt = (1u << lane) - 1u;
    for (long long base = begin; base < end; base += 32) {
        const long long a = base + lane;
        const int e = a < end ? expert_idx[a] : -1;
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        if (e >= 0 && (peers & lt) == 0) s_hist[warp][e] += __popc(peers);
        __syncwarp();
    }
    __syncthreads();
    for (int e = threadIdx.x; e < E; e += blockDim.x) {
        int run = offsets[e] + block_base[(long long)blockIdx.x * E + e];
#pragma unroll
        for (int w = 0; w < kWarps; ++w) {
            const int c = s_hist[w][e];
            s_hist[w][e] = run;
            run += c;
        }
    }
    __syncthreads();
    for (long long base = begin; base < end; base += 32) {
        const long long a = base + lane;
        const int e = a < end ? expert_idx[a] : -1;
        const unsigned peers = __match_any_sync(0xffffffffu, e);
        int dest = -1;
        if (e >= 0) dest = s_hist[warp][e] + __popc(peers & lt);
        __syncwarp();
        if (e >= 0 && (peers & lt) == 0) s_hist[warp][e] += __popc(peers);
        __syncwarp();
        if (e >= 0) {
            dest_row[a] = dest;
            row_source[dest] = (int)a;
        }
    }
}

__global__ void route_export_kernel(const int* __restrict__ expert_idx, const int* __restrict__ dest_row,
                                    const int* __restrict__ offsets, const int* __restrict__ counts,
                                    long long* indices, long long* ids, long long* slots,
                                    long long* locations, long long* counts64, long long A, int E,
                                    int k, long long capacity) {
    const long long a = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (a < E && counts64) counts64[a] = counts[a];
    if (a >= A) return;
    const int e = expert_idx[a];
    const long long loc = dest_row[a] - offsets[e];
    if (indices) indices[a] = e;
    if (locations) locations[a] = loc;
    if (ids) ids[e * capacity + loc] = a / k;
    if (slots) slots[e * capacity + loc] = a % k;
}

// ---- routing backward: one warp per token row -------------------------------------------------
__global__ void __launch_bounds__(256)
route_backward_kernel(const float* __restrict__ probs, const float* __restrict__ gate_w,
                      const int* __restrict__ expert_idx, const float* __restrict__ util,
                      const float* __restrict__ grad_w, const float* __restrict__ grad_aux,
                      float* __restrict__ d_scores, long long T, int E, int k) {
    const int lane = threadIdx.x & 31;
    const long long row = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (row >= T) return;
    const float ga = grad_aux ? grad_aux[0] * (float)E / (float)T : 0.f;
    float center_aux = 0.f;
    if (grad_aux) {
        for (int e = lane; e < E; e += 32) center_aux += probs[row * E + e] * util[e];
        center_aux = warp_sum(center_aux);
    }
    float center = 0.f;
    if (grad_w)
        for (int s = 0; s < k; ++s) center += grad_w[row * k + s] * gate_w[row * k + s];
    for (int e = lane; e < E; e += 32) {
        float value = 0.f;
        if (grad_aux) value = ga * probs[row * E + e] * (util[e] - center_aux);
        if (grad_w)
            for (int s = 0; s < k; ++s)
                if (expert_idx[row * k + s] == e)
                    value += gate_w[row * k + s] * (grad_w[row * k + s] - center);
        d_scores[row * E + e] = value;
    }
}

// need_scratch: the three block tables are only used while the routing itself runs (qmoe_route); every
// consumer of a finished route accepts null there, so a route filled by qmoe_route_static can be passed on.
int check_route(const qmoe_route_t* r, bool need_scratch) {
    if (!r) return fail_arg("route is null");
    if (r->tokens <= 0) return fail_arg("tokens must be positive (got %lld)", (long long)r->tokens);
    if (r->experts <= 0 || r->experts > kMaxExperts)
        return fail_arg("experts must be in [1, %d] (got %d)", kMaxExperts, r->experts);
    // top_k <= experts is a property of routing.  The consumers of a finished route also take the expert-side view an
    // expert-parallel rank builds of its local experts, which can be fewer than top_k (8 experts top-2 over 8 ranks).
    if (r->top_k <= 0 || r->top_k > kMaxTopK || (need_scratch && r->top_k > r->experts))
        return fail_arg("top_k must be in [1, min(experts, %d)] (got %d)", kMaxTopK, r->top_k);
    if (r->tokens * r->top_k > (1ll << 30)) return fail_arg("tokens * top_k exceeds 2^30");
    if (r->rows_bound < qmoe_rows_bound(r->tokens, r->experts, r->top_k))
        return fail_arg("rows_bound %lld is smaller than qmoe_rows_bound()", (long long)r->rows_bound);
    if (!r->probs || !r->gate_weights || !r->expert_index || !r->dest_row || !r->row_source ||
        !r->counts || !r->offsets || !r->tile_expert || !r->meta || !r->utilization || !r->aux)
        return fail_arg("route has a null table address");
    if (need_scratch && (!r->block_counts || !r->block_base || !r->block_colsum))
        return fail_arg("route has a null scratch table address (block_counts / block_base / block_colsum)");
    return 0;
}

}  // namespace

int route_check(const qmoe_route_t* r) { return check_route(r, false); }

}  // namespace qmoe

using namespace qmoe;

extern "C" int64_t qmoe_rows_bound(int64_t tokens, int32_t experts, int32_t top_k) {
    const int64_t a = tokens * top_k + (int64_t)experts * (kRowPad - 1);
    return (a + kRowPad - 1) / kRowPad * kRowPad;
}

extern "C" int64_t qmoe_route_blocks(int64_t tokens) {
    return (tokens + kRouteRowsPerBlock - 1) / kRouteRowsPerBlock;
}

extern "C" int qmoe_route(const qmoe_route_t* r, uint64_t scores, uint64_t stream_) {
    if (int rc = check_route(r, true)) return rc;
    if (!scores) return fail_arg("scores is null");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_ROUTE, stream);
    const int nblk = (int)qmoe_route_blocks(r->tokens);
    const long long T = r->tokens;
    const int E = r->experts, k = r->top_k;
    QMOE_CUDA(cudaMemsetAsync((void*)r->row_source, 0xff, (size_t)r->rows_bound * sizeof(int), stream));
    const float* sc = (const float*)scores;
    float* probs = (float*)r->probs;
    float* gw = (float*)r->gate_weights;
    int* eidx = (int*)r->expert_index;
    int* bc = (int*)r->block_counts;
    float* bs = (float*)r->block_colsum;
    const int epl = (E + 31) / 32;
    if (epl <= 1) route_topk_kernel<1><<<nblk, kWarps * 32, 0, stream>>>(sc, probs, gw, eidx, bc, bs, T, E, k);
    else if (epl <= 2) route_topk_kernel<2><<<nblk, kWarps * 32, 0, stream>>>(sc, probs, gw, eidx, bc, bs, T, E, k);
    else if (epl <= 4) route_topk_kernel<4><<<nblk, kWarps * 32, 0, stream>>>(sc, probs, gw, eidx, bc, bs, T, E, k);
    else route_topk_kernel<8><<<nblk, kWarps * 32, 0, stream>>>(sc, probs, gw, eidx, bc, bs, T, E, k);
    QMOE_LAUNCH_CHECK("route_topk_kernel");
    route_scan_kernel<<<1, kScanThreads, 0, stream>>>(bc, bs, (int*)r->block_base, (int*)r->counts,
                                                      (int*)r->offsets, (int*)r->tile_expert,
                                                      (int*)r->meta, (float*)r->utilization,
                                                      (float*)r->aux, nblk, T, E, k);
    QMOE_LAUNCH_CHECK("route_scan_kernel");
    route_pack_kernel<<<nblk, kWarps * 32, 0, stream>>>(eidx, (const int*)r->block_base,
                                                        (const int*)r->offsets, (int*)r->dest_row,
                                                        (int*)r->row_source, T, E, k);
    QMOE_LAUNCH_CHECK("route_pack_kernel");
    return 0;
}

extern "C" int qmoe_route_export_i64(const qmoe_route_t* r, uint64_t indices, uint64_t ids, uint64_t slots,
                                     uint64_t locations, uint64_t counts, int64_t capacity,
                                     uint64_t stream_) {
    if (int rc = check_route(r, false)) return rc;
    const long long A = r->tokens * r->top_k;
    if ((ids || slots) && capacity < A) return fail_arg("capacity %lld is smaller than tokens*top_k", (long long)capacity);
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_OTHER, stream);
    const long long n = A > r->experts ? A : r->experts;
    route_export_kernel<<<ceil_div(n, 256), 256, 0, stream>>>(
        (const int*)r->expert_index, (const int*)r->dest_row, (const int*)r->offsets,
        (const int*)r->counts, (long long*)indices, (long long*)ids, (long long*)slots,
        (long long*)locations, (long long*)counts, A, r->experts, r->top_k, capacity);
    QMOE_LAUNCH_CHECK("route_export_kernel");
    return 0;
}

extern "C" int qmoe_route_backward(const qmoe_route_t* r, uint64_t grad_weights, uint64_t grad_aux,
                                   uint64_t d_scores, uint64_t stream_) {
    if (int rc = check_route(r, false)) return rc;
    if (!d_scores) return fail_arg("d_scores is null");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_ROUTE_BWD, stream);
    if (!grad_weights && !grad_aux) {
        QMOE_CUDA(cudaMemsetAsync((void*)d_scores, 0, (size_t)r->tokens * r->experts * sizeof(float), stream));
        return 0;
    }
    route_backward_kernel<<<ceil_div(r->tokens, 8), 256, 0, stream>>>(
        (const float*)r->probs, (const float*)r->gate_weights, (const int*)r->expert_index,
        (const float*)r->utilization, (const float*)grad_weights, (const float*)grad_aux,
        (float*)d_scores, r->tokens, r->experts, r->top_k);
    QMOE_LAUNCH_CHECK("route_backward_kernel");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// qmoe_route_static: qmoe_route for callers that cannot supply scratch memory.
//
// qmoe_route needs three scratch tables (block_counts, block_base, block_colsum) besides its inputs
// and outputs, and expects the caller to allocate them.  Some hosts cannot: a serving loop that
// must never call cudaMalloc on its request path (the call synchronises the whole device), a
// plug-in host that was handed a fixed set of buffers at start-up and has no allocator of its own
// to reach for more, or a runtime whose memory pool is private to it.  For them the three tables
// live in the fixed device array below, which every GPU that loads this library keeps resident
// until the process exits (1.5 MiB).  The caller still passes every input and output table.
//
// Limit: blocks * experts <= kStaticRouteEntries, where blocks = qmoe_route_blocks(tokens); larger
// problems are rejected with an argument error and must use qmoe_route.
//
// The array is shared by all calls and keeps whatever the previous call left in it.  That is
// harmless here because the first routing kernel writes every entry it later reads (one row per
// block, all experts), so nothing has to start at zero and nothing is cleared.  It also means two
// calls whose kernels overlap on the GPU (different streams, or different host threads) race on the
// array: issue calls to this entry point on one stream at a time per device.
//
// The first call on a device looks up the array's device address (cudaGetSymbolAddress, checked)
// with that device current, and remembers it; make that first call before starting any stream
// capture.  The remembered address is written without a lock: two host threads that make the first
// call at the same moment both look the address up and store the same value.  No cudaMalloc, cudaFree or allocating library routine is called on any path.
namespace {
constexpr long long kStaticRouteEntries = 131072;  // entries per table (blocks * experts)
static __device__ __align__(256) unsigned char g_route_scratch[3 * kStaticRouteEntries * 4];
constexpr int kMaxDevices = 64;
void* g_route_scratch_address[kMaxDevices] = {nullptr};  // device address per device, looked up once
}  // namespace

extern "C" int qmoe_route_static(const qmoe_route_t* r, uint64_t scores, uint64_t stream_) {
    if (!r) return fail_arg("route is null");
    if (r->tokens <= 0 || r->experts <= 0) return fail_arg("route_static: tokens and experts must be positive");
    const long long entries = qmoe_route_blocks(r->tokens) * (long long)r->experts;
    if (entries > kStaticRouteEntries)
        return fail_arg("route_static: %lld blocks x %d experts = %lld scratch entries exceed the built-in %lld; "
                        "use qmoe_route with caller-allocated scratch",
                        (long long)qmoe_route_blocks(r->tokens), r->experts, entries, kStaticRouteEntries);
    int device = 0;
    QMOE_CUDA(cudaGetDevice(&device));
    if (device < 0 || device >= kMaxDevices) return fail_arg("route_static: device index %d is out of range", device);
    if (!g_route_scratch_address[device]) {
        // In host code `g_route_scratch` only stands for the symbol; the address kernels can use
        // has to be asked for, once per device, while that device is current.
        void* address = nullptr;
        QMOE_CUDA(cudaGetSymbolAddress(&address, g_route_scratch));
        if (!address) { set_error("route_static: the scratch array has no device address"); return QMOE_ERR_STATE; }
        g_route_scratch_address[device] = address;
    }
    unsigned char* base = (unsigned char*)g_route_scratch_address[device];
    qmoe_route_t with_scratch = *r;
    with_scratch.block_counts = (uint64_t)base;
    with_scratch.block_base = (uint64_t)(base + kStaticRouteEntries * 4);
    with_scratch.block_colsum = (uint64_t)(base + 2 * kStaticRouteEntries * 4);
    return qmoe_route(&with_scratch, scores, stream_);
}
