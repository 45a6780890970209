// Expert parallelism over NCCL (NVLink 5 / NVSwitch): one process per GPU, tokens sharded by rank,
// experts sharded by rank in contiguous blocks.  The upstream project is single-GPU
// (src/qutai/backends/cuda_runtime.py:82, :105); this file is new functionality around the same
// layer semantics: the rows an expert receives are ordered (source rank, local (token, slot) order),
// which with contiguous token shards IS the upstream global (token, slot) order
// (src/qutai/backends/cuda/lm.cu:353-383).
//
// NCCL is opened at run time (dlopen of libnccl.so.2): when the host process already carries an
// NCCL (e.g. the one bundled with torch) the same library instance is used.  Nothing here waits on
// flags of its own: all cross-GPU ordering comes from NCCL's stream semantics.
#include <dlfcn.h>
#include <nccl.h>

#include <mutex>

#include "common.cuh"

namespace qmoe {
namespace {

struct NcclApi {
    void* handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*CommInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    const char* (*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*AllGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*AllReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Send)(const void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*Recv)(void*, size_t, ncclDataType_t, int, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*GroupStart)() = nullptr;
    ncclResult_t (*GroupEnd)() = nullptr;
};

NcclApi g_nccl;
std::mutex g_ep_mutex;
ncclComm_t g_comm = nullptr;
int g_rank = 0, g_world = 0;

int load_nccl() {
    if (g_nccl.handle) return 0;
    const char* names[] = {getenv("QUTAI_MOE_NCCL"), "libnccl.so.2", "libnccl.so"};
    for (const char* name : names) {
        if (!name || !*name) continue;
        g_nccl.handle = dlopen(name, RTLD_NOW | RTLD_GLOBAL);
        if (g_nccl.handle) break;
    }
    if (!g_nccl.handle) { set_error("cannot open libnccl.so.2: %s", dlerror()); return QMOE_ERR_STATE; }
#define LOAD(field, symbol)                                                                  \
    *(void**)(&g_nccl.field) = dlsym(g_nccl.handle, symbol);                                 \
    if (!g_nccl.field) { set_error("libnccl has no symbol %s", symbol); g_nccl.handle = nullptr; return QMOE_ERR_STATE; }
    LOAD(GetUniqueId, "ncclGetUniqueId") LOAD(CommInitRank, "ncclCommInitRank") LOAD(CommDestroy, "ncclCommDestroy")
    LOAD(CommAbort, "ncclCommAbort") LOAD(GetErrorString, "ncclGetErrorString") LOAD(AllGather, "ncclAllGather")
    LOAD(AllReduce, "ncclAllReduce") LOAD(Send, "ncclSend") LOAD(Recv, "ncclRecv") LOAD(GroupStart, "ncclGroupStart")
    LOAD(GroupEnd, "ncclGroupEnd")
#undef LOAD
    return 0;
}

int check_nccl(ncclResult_t code, const char* what) {
    if (code == ncclSuccess) return 0;
    set_error("%s failed: %s", what, g_nccl.GetErrorString ? g_nccl.GetErrorString(code) : "NCCL error");
    return 1000 + (int)code;
}
#define QMOE_NCCL(expr)                                  \
    do {                                                 \
        int _rc = check_nccl((expr), #expr);             \
        if (_rc) return _rc;                             \
    } while (0)

int need_comm() {
    if (!g_comm) { set_error("expert parallelism is not initialised (call qmoe_ep_init first)"); return QMOE_ERR_STATE; }
    return 0;
}

// local statistics of one rank: counts[E] and the per-expert probability column sums (as float bits)
__global__ void __launch_bounds__(kMaxExperts)
ep_stats_kernel(const int* __restrict__ counts, const float* __restrict__ block_colsum, int nblk, int E, int* __restrict__ stats) {
    const int e = threadIdx.x;
    if (e >= E) return;
    double cs = 0.0;
    for (int b = 0; b < nblk; ++b) cs += (double)block_colsum[(long long)b * E + e];  // fixed order
    stats[e] = counts[e];
    stats[E + e] = __float_as_int((float)cs);
}

// From the gathered [world, 2E] statistics: global utilisation and auxiliary loss (written into the
// token-side route), and the dispatched-layout tables of this rank's experts (expert-side route).
__global__ void __launch_bounds__(kMaxExperts)
ep_plan_kernel(const int* __restrict__ stats_all, int world, int rank, int E, int E_loc, long long T_global, int k,
               float* __restrict__ util, float* __restrict__ aux, int* __restrict__ x_counts, int* __restrict__ x_offsets,
               int* __restrict__ x_tile_expert, int* __restrict__ x_meta) {
    __shared__ double s_part[kMaxExperts];
    __shared__ int s_cnt[kMaxExperts];
    __shared__ int s_off[kMaxExperts + 1];
    const int e = threadIdx.x;
    const double A = (double)T_global * k;
    if (e < E) {
        long long count = 0;
        double cs = 0.0;
        for (int p = 0; p < world; ++p) {  // fixed rank order: every rank computes the same bits
            count += stats_all[(long long)p * 2 * E + e];
            cs += (double)__int_as_float(stats_all[(long long)p * 2 * E + E + e]);
        }
        util[e] = (float)((double)count / A);
        s_part[e] = ((double)count / A) * cs / (double)T_global;
        if (e >= rank * E_loc && e < (rank + 1) * E_loc) {
            s_cnt[e - rank * E_loc] = (int)count;
            x_counts[e - rank * E_loc] = (int)count;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        double total = 0.0;
        for (int i = 0; i < E; ++i) total += s_part[i];
        aux[0] = (float)((double)E * total);
        int off = 0;
        for (int i = 0; i < E_loc; ++i) {
            s_off[i] = off;
            x_offsets[i] = off;
            off += (s_cnt[i] + kRowPad - 1) / kRowPad * kRowPad;
        }
        s_off[E_loc] = off;
        x_offsets[E_loc] = off;
        x_meta[0] = off;
        x_meta[1] = off / kRowPad;
        x_meta[2] = 0;
        x_meta[3] = 0;
    }
    __syncthreads();
    if (e < E_loc)
        for (int t = s_off[e] / kRowPad; t < s_off[e + 1] / kRowPad; ++t) x_tile_expert[t] = e;
}

// zero the pad rows [offsets[e] + counts[e], offsets[e + 1]) of every expert group
__global__ void __launch_bounds__(256)
ep_zero_pads_kernel(uint4* __restrict__ buf, const int* __restrict__ offsets, const int* __restrict__ counts, int E,
                    long long row_vecs) {
    const int e = blockIdx.y;
    if (e >= E) return;
    const long long first = (long long)(offsets[e] + counts[e]) * row_vecs, last = (long long)offsets[e + 1] * row_vecs;
    for (long long i = first + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < last; i += (long long)gridDim.x * blockDim.x)
        buf[i] = make_uint4(0, 0, 0, 0);
}

}  // namespace
}  // namespace qmoe

using namespace qmoe;

extern "C" int qmoe_ep_unique_id(void* id128) {
    if (!id128) return fail_arg("ep_unique_id: buffer is null");
    std::lock_guard<std::mutex> lock(g_ep_mutex);
    if (int rc = load_nccl()) return rc;
    static_assert(sizeof(ncclUniqueId) == 128, "NCCL unique id is 128 bytes");
    QMOE_NCCL(g_nccl.GetUniqueId((ncclUniqueId*)id128));
    return 0;
}

extern "C" int qmoe_ep_init(int32_t rank, int32_t world, const void* id128) {
    if (!id128 || world <= 0 || rank < 0 || rank >= world) return fail_arg("ep_init: bad rank/world or null id");
    std::lock_guard<std::mutex> lock(g_ep_mutex);
    if (g_comm) { set_error("expert parallelism is already initialised"); return QMOE_ERR_STATE; }
    if (int rc = load_nccl()) return rc;
    ncclUniqueId id;
    memcpy(&id, id128, sizeof(id));
    QMOE_NCCL(g_nccl.CommInitRank(&g_comm, world, id, rank));
    g_rank = rank;
    g_world = world;
    return 0;
}

extern "C" int qmoe_ep_finalize(int32_t abort_communicator) {
    std::lock_guard<std::mutex> lock(g_ep_mutex);
    if (!g_comm) return 0;
    ncclComm_t comm = g_comm;
    g_comm = nullptr;
    g_world = 0;
    // abort does not wait for outstanding collectives: the path a host takes after it learned
    // (by its own means) that a peer is gone
    QMOE_NCCL(abort_communicator ? g_nccl.CommAbort(comm) : g_nccl.CommDestroy(comm));
    return 0;
}

extern "C" int qmoe_ep_info(int32_t* rank, int32_t* world) {
    if (rank) *rank = g_rank;
    if (world) *world = g_world;
    return 0;
}

extern "C" int qmoe_ep_gather_stats(const qmoe_route_t* r, uint64_t stats_local, uint64_t stats_all, void* host_stats,
                                    uint64_t stream_) {
    if (int rc = route_check(r)) return rc;
    if (int rc = need_comm()) return rc;
    if (!stats_local || !stats_all) return fail_arg("ep_gather_stats: null buffer");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_OTHER, stream);
    const int E = r->experts;
    ep_stats_kernel<<<1, kMaxExperts, 0, stream>>>((const int*)r->counts, (const float*)r->block_colsum,
                                                    (int)qmoe_route_blocks(r->tokens), E, (int*)stats_local);
    QMOE_LAUNCH_CHECK("ep_stats_kernel");
    QMOE_NCCL(g_nccl.AllGather((const void*)stats_local, (void*)stats_all, (size_t)2 * E, ncclInt32, g_comm, stream));
    if (host_stats)
        QMOE_CUDA(cudaMemcpyAsync(host_stats, (const void*)stats_all, (size_t)g_world * 2 * E * sizeof(int),
                                  cudaMemcpyDeviceToHost, stream));
    return 0;
}

extern "C" int qmoe_ep_plan(uint64_t stats_all, const qmoe_route_t* token_route, const qmoe_route_t* expert_route,
                            int64_t tokens_global, uint64_t stream_) {
    if (int rc = route_check(token_route)) return rc;
    if (int rc = route_check(expert_route)) return rc;
    if (int rc = need_comm()) return rc;
    if (!stats_all) return fail_arg("ep_plan: stats_all is null");
    const int E = token_route->experts, E_loc = expert_route->experts;
    if (E_loc * g_world != E) return fail_arg("ep_plan: %d local experts x %d ranks != %d experts", E_loc, g_world, E);
    if (expert_route->rows_bound < qmoe_rows_bound(tokens_global, E_loc, token_route->top_k))
        return fail_arg("ep_plan: expert-side rows_bound is too small for %lld global tokens", (long long)tokens_global);
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_OTHER, stream);
    ep_plan_kernel<<<1, kMaxExperts, 0, stream>>>((const int*)stats_all, g_world, g_rank, E, E_loc, tokens_global,
                                                   token_route->top_k, (float*)token_route->utilization,
                                                   (float*)token_route->aux, (int*)expert_route->counts,
                                                   (int*)expert_route->offsets, (int*)expert_route->tile_expert,
                                                   (int*)expert_route->meta);
    QMOE_LAUNCH_CHECK("ep_plan_kernel");
    return 0;
}

extern "C" int qmoe_ep_zero_pad_rows(const qmoe_route_t* expert_route, uint64_t buf, int32_t dtype, int64_t width,
                                     uint64_t stream_) {
    if (int rc = route_check(expert_route)) return rc;
    if (!buf || width <= 0) return fail_arg("ep_zero_pad_rows: null buffer or bad width");
    const long long row_bytes = width * (dtype == QMOE_BF16 ? 2 : 4);
    if (row_bytes % 16 || buf & 15u) return fail_arg("ep_zero_pad_rows: rows must be multiples of 16 bytes");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_OTHER, stream);
    dim3 grid(8, expert_route->experts);
    ep_zero_pads_kernel<<<grid, 256, 0, stream>>>((uint4*)buf, (const int*)expert_route->offsets,
                                                  (const int*)expert_route->counts, expert_route->experts, row_bytes / 16);
    QMOE_LAUNCH_CHECK("ep_zero_pads_kernel");
    return 0;
}

extern "C" int qmoe_ep_exchange(uint64_t send_buf, const qmoe_ep_segment_t* sends, int32_t n_sends, uint64_t recv_buf,
                                const qmoe_ep_segment_t* recvs, int32_t n_recvs, int64_t width, int32_t dtype,
                                uint64_t stream_) {
    if (int rc = need_comm()) return rc;
    if (n_sends < 0 || n_recvs < 0 || (n_sends && (!sends || !send_buf)) || (n_recvs && (!recvs || !recv_buf)))
        return fail_arg("ep_exchange: null buffer or segment list");
    if (width <= 0 || (dtype != QMOE_BF16 && dtype != QMOE_F32)) return fail_arg("ep_exchange: bad width or dtype");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_EXCHANGE, stream);
    const size_t item = dtype == QMOE_BF16 ? 2 : 4;
    const ncclDataType_t type = dtype == QMOE_BF16 ? ncclBfloat16 : ncclFloat32;
    for (int i = 0; i < n_sends; ++i)
        if (sends[i].peer < 0 || sends[i].peer >= g_world || sends[i].rows < 0 || sends[i].offset_rows < 0)
            return fail_arg("ep_exchange: send segment %d is invalid", i);
    for (int i = 0; i < n_recvs; ++i)
        if (recvs[i].peer < 0 || recvs[i].peer >= g_world || recvs[i].rows < 0 || recvs[i].offset_rows < 0)
            return fail_arg("ep_exchange: receive segment %d is invalid", i);
    // Segments that stay on this rank are plain device-to-device copies, matched in list order
    // like any other pair; only rows that really change GPU go through NCCL.
    {
        int r = 0;
        for (int i = 0; i < n_sends; ++i) {
            if (sends[i].peer != g_rank || !sends[i].rows) continue;
            while (r < n_recvs && (recvs[r].peer != g_rank || !recvs[r].rows)) ++r;
            if (r >= n_recvs || recvs[r].rows != sends[i].rows)
                return fail_arg("ep_exchange: local send segment %d has no matching local receive segment", i);
            QMOE_CUDA(cudaMemcpyAsync((char*)recv_buf + (size_t)recvs[r].offset_rows * width * item,
                                      (const char*)send_buf + (size_t)sends[i].offset_rows * width * item,
                                      (size_t)sends[i].rows * width * item, cudaMemcpyDeviceToDevice, stream));
            ++r;
        }
    }
    QMOE_NCCL(g_nccl.GroupStart());
    int rc = 0;
    for (int i = 0; i < n_sends && !rc; ++i)
        if (sends[i].rows && sends[i].peer != g_rank)
            rc = check_nccl(g_nccl.Send((const char*)send_buf + (size_t)sends[i].offset_rows * width * item,
                                        (size_t)sends[i].rows * width, type, sends[i].peer, g_comm, stream), "ncclSend");
    for (int i = 0; i < n_recvs && !rc; ++i)
        if (recvs[i].rows && recvs[i].peer != g_rank)
            rc = check_nccl(g_nccl.Recv((char*)recv_buf + (size_t)recvs[i].offset_rows * width * item,
                                        (size_t)recvs[i].rows * width, type, recvs[i].peer, g_comm, stream), "ncclRecv");
    const int end = check_nccl(g_nccl.GroupEnd(), "ncclGroupEnd");
    return rc ? rc : end;
}

extern "C" int qmoe_ep_all_reduce_f32(uint64_t buf, int64_t n, uint64_t stream_) {
    if (int rc = need_comm()) return rc;
    if (!buf || n < 0) return fail_arg("ep_all_reduce_f32: null buffer or negative size");
    if (n == 0) return 0;
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_OTHER, stream);
    QMOE_NCCL(g_nccl.AllReduce((const void*)buf, (void*)buf, (size_t)n, ncclFloat32, ncclSum, g_comm, stream));
    return 0;
}
