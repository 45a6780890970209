// Expert parallelism over NCCL (NVLink 5 / NVSwitch): one process per GPU, tokens sharded by rank,
// experts sharded by rank in contiguous blocks.  The upstream project is single-GPU
// (src/qutai/backends/cuda_runtime.py:82, :105); this file is new functionality around the same
// layer semantics: the rows an expert receives are ordered (source rank, local (token, slot) order),
// which with contiguous token shards IS the upstream global (token, slot) order
// (src/qutai/backends/cuda/lm.cu:353-383).
//
// NCCL is opened at run time (dlopen of libnccl.so.2): when the host process already carries an
// NCCL (e.g. the one bundled with torch) the same library instance is used.  With the NCCL transport all
// cross-GPU ordering comes from NCCL's stream semantics; the direct transport orders the ranks with
// ep_flag_barrier_kernel, whose wait on the peers' flags is bounded and reports a status instead of hanging.
#include <dlfcn.h>
#include <nccl.h>

#include <atomic>
#include <initializer_list>
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
    if (!r->block_colsum) return fail_arg("ep_gather_stats: route.block_colsum is null (a route filled by qmoe_route_static keeps its column sums inside the library)");
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
    TimedScope timed(KC_ALL_REDUCE, stream);
    QMOE_NCCL(g_nccl.AllReduce((const void*)buf, (void*)buf, (size_t)n, ncclFloat32, ncclSum, g_comm, stream));
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Direct transport: rows are pushed into the destination GPU's buffer with plain 16-byte stores
// over NVLink (peer memory mapped through CUDA IPC), one warp per row.  Sizes and destinations are
// computed on the device from the gathered counts, so the host never has to read them.  Cross-GPU
// ordering after each push is either a tiny NCCL collective (qmoe_ep_barrier) or the flag barrier further
// down (qmoe_ep_flag_barrier), the only kernel here that waits on another GPU, for a bounded time.
// ---------------------------------------------------------------------------------------------
namespace qmoe {
namespace {

constexpr int kMaxPeers = QMOE_EP_MAX_RANKS;
constexpr int kRetRankShift = 26;  // return address = (source rank << 26) | source row

struct PeerTable {
    uint4* buffer[kMaxPeers];
    int* ret[kMaxPeers];
};

// dest_base[e]: row, inside the owner's expert-side layout, where THIS rank's rows for expert e start
__global__ void __launch_bounds__(kMaxExperts)
ep_dest_base_kernel(const int* __restrict__ stats_all, int world, int rank, int E, int E_loc, int* __restrict__ dest_base) {
    __shared__ int s_total[kMaxExperts];
    const int e = threadIdx.x;
    if (e < E) {
        int total = 0;
        for (int p = 0; p < world; ++p) total += stats_all[(long long)p * 2 * E + e];
        s_total[e] = total;
    }
    __syncthreads();
    if (e >= E) return;
    int off = 0;
    for (int j = (e / E_loc) * E_loc; j < e; ++j) off += (s_total[j] + kRowPad - 1) / kRowPad * kRowPad;
    for (int q = 0; q < rank; ++q) off += stats_all[(long long)q * 2 * E + e];
    dest_base[e] = off;
}

// Token side -> expert side.  Row r of the local dispatched layout (expert e = tile_expert[r / 128],
// index i = r - offsets[e] inside the expert, a real row when i < counts[e]) goes to rank e / E_loc,
// row dest_base[e] + i, and its return address is recorded next to it.
__global__ void __launch_bounds__(256, 6)
ep_push_dispatch_kernel(const uint4* __restrict__ src, long long row_vecs, const int* __restrict__ tile_expert,
                        const int* __restrict__ offsets, const int* __restrict__ counts, const int* __restrict__ meta,
                        const int* __restrict__ dest_base, int E_loc, int rank, PeerTable peers) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    const int rows = meta[0];
    for (long long r = warp; r < rows; r += nwarps) {
        const int e = tile_expert[r / kRowPad];
        const int i = (int)r - offsets[e];
        if (i >= counts[e]) continue;  // pad row: nothing to send
        const int p = e / E_loc;
        const long long dest = (long long)dest_base[e] + i;
        const uint4* s = src + r * row_vecs;
        uint4* d = peers.buffer[p] + dest * row_vecs;
        long long c = lane;
        for (; c + 96 < row_vecs; c += 128) {
            const uint4 v0 = s[c], v1 = s[c + 32], v2 = s[c + 64], v3 = s[c + 96];
            d[c] = v0; d[c + 32] = v1; d[c + 64] = v2; d[c + 96] = v3;
        }
        for (; c < row_vecs; c += 32) d[c] = s[c];
        if (lane == 0 && peers.ret[p]) peers.ret[p][dest] = (rank << kRetRankShift) | (int)r;
    }
    __threadfence_system();
}

// Expert side -> token side.  Row j of the local expert-side layout (a real row when it lies in
// [offsets[x], offsets[x] + counts[x])) goes back to the rank and row recorded in ret[j].
__global__ void __launch_bounds__(256, 6)
ep_push_return_kernel(const uint4* __restrict__ src, long long row_vecs, const int* __restrict__ tile_expert,
                      const int* __restrict__ offsets, const int* __restrict__ counts, const int* __restrict__ meta,
                      const int* __restrict__ ret, int expert_begin, int expert_end, PeerTable peers) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    const int rows = meta[0];
    for (long long j = warp; j < rows; j += nwarps) {
        const int x = tile_expert[j / kRowPad];
        if (x < expert_begin || x >= expert_end || (int)j - offsets[x] >= counts[x]) continue;
        const int address = ret[j];
        const int q = address >> kRetRankShift;
        const long long dest = address & ((1 << kRetRankShift) - 1);
        const uint4* s = src + j * row_vecs;
        uint4* d = peers.buffer[q] + dest * row_vecs;
        long long c = lane;
        for (; c + 96 < row_vecs; c += 128) {
            const uint4 v0 = s[c], v1 = s[c + 32], v2 = s[c + 64], v3 = s[c + 96];
            d[c] = v0; d[c + 32] = v1; d[c + 64] = v2; d[c + 96] = v3;
        }
        for (; c < row_vecs; c += 32) d[c] = s[c];
    }
    __threadfence_system();
}

int check_peers(const qmoe_ep_peers_t* peers, bool need_ret) {
    if (!peers) return fail_arg("peers is null");
    if (peers->world <= 0 || peers->world > kMaxPeers || peers->rank < 0 || peers->rank >= peers->world)
        return fail_arg("peers: world must be in [1, %d] and rank inside it", kMaxPeers);
    for (int p = 0; p < peers->world; ++p) {
        if (!peers->buffer[p] || (peers->buffer[p] & 15u)) return fail_arg("peers: buffer of rank %d is null or misaligned", p);
        if (need_ret && !peers->ret[p]) return fail_arg("peers: return table of rank %d is null", p);
    }
    return 0;
}

PeerTable make_table(const qmoe_ep_peers_t* peers, bool with_ret) {
    PeerTable t = {};
    for (int p = 0; p < peers->world; ++p) {
        t.buffer[p] = (uint4*)peers->buffer[p];
        t.ret[p] = with_ret ? (int*)peers->ret[p] : nullptr;
    }
    return t;
}

// blocks_per_sm: 0 = fill the GPU (8 blocks of 256 threads per SM); a push that is meant to run beside
// a tensor-core kernel asks for 1, so that both fit on every SM at the same time
int push_grid(long long rows, int blocks_per_sm) {
    long long blocks = (rows + 7) / 8;
    const long long cap = (long long)sm_count() * (blocks_per_sm > 0 && blocks_per_sm < 8 ? blocks_per_sm : 8);
    return (int)(blocks > cap ? cap : (blocks < 1 ? 1 : blocks));
}

}  // namespace
}  // namespace qmoe

extern "C" int qmoe_set_device(int32_t device) {
    QMOE_CUDA(cudaSetDevice(device));
    return 0;
}

extern "C" int qmoe_ep_ipc_export(uint64_t address, void* handle64) {
    if (!address || !handle64) return fail_arg("ep_ipc_export: null argument");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "CUDA IPC handles are 64 bytes");
    QMOE_CUDA(cudaIpcGetMemHandle((cudaIpcMemHandle_t*)handle64, (void*)address));
    return 0;
}

extern "C" int qmoe_ep_ipc_open(const void* handle64, uint64_t* address) {
    if (!handle64 || !address) return fail_arg("ep_ipc_open: null argument");
    cudaIpcMemHandle_t handle;
    memcpy(&handle, handle64, sizeof(handle));
    void* p = nullptr;
    QMOE_CUDA(cudaIpcOpenMemHandle(&p, handle, cudaIpcMemLazyEnablePeerAccess));
    *address = (uint64_t)p;
    return 0;
}

extern "C" int qmoe_ep_ipc_close(uint64_t address) {
    if (!address) return 0;
    QMOE_CUDA(cudaIpcCloseMemHandle((void*)address));
    return 0;
}

extern "C" int qmoe_ep_barrier(uint64_t scratch_i32, uint64_t stream_) {
    if (int rc = need_comm()) return rc;
    if (!scratch_i32) return fail_arg("ep_barrier: scratch is null");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_BARRIER, stream);
    QMOE_NCCL(g_nccl.AllReduce((const void*)scratch_i32, (void*)scratch_i32, 1, ncclInt32, ncclSum, g_comm, stream));
    return 0;
}

extern "C" int qmoe_ep_dest_base(uint64_t stats_all, int32_t experts, int32_t local_experts, uint64_t dest_base,
                                 uint64_t stream_) {
    if (int rc = need_comm()) return rc;
    if (!stats_all || !dest_base) return fail_arg("ep_dest_base: null buffer");
    if (experts <= 0 || experts > kMaxExperts || local_experts * g_world != experts)
        return fail_arg("ep_dest_base: %d local experts x %d ranks != %d experts", local_experts, g_world, experts);
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_OTHER, stream);
    ep_dest_base_kernel<<<1, kMaxExperts, 0, stream>>>((const int*)stats_all, g_world, g_rank, experts, local_experts,
                                                        (int*)dest_base);
    QMOE_LAUNCH_CHECK("ep_dest_base_kernel");
    return 0;
}

extern "C" int qmoe_ep_push_dispatch(const qmoe_route_t* token_route, uint64_t dest_base, uint64_t src,
                                     const qmoe_ep_peers_t* peers, int32_t write_return_addresses, int32_t blocks_per_sm,
                                     int32_t dtype, int64_t width, uint64_t stream_) {
    if (int rc = route_check(token_route)) return rc;
    if (int rc = check_peers(peers, write_return_addresses != 0)) return rc;
    if (!dest_base || !src || (src & 15u)) return fail_arg("ep_push_dispatch: null or misaligned buffer");
    const long long row_bytes = width * (dtype == QMOE_BF16 ? 2 : 4);
    if (width <= 0 || row_bytes % 16) return fail_arg("ep_push_dispatch: rows must be multiples of 16 bytes");
    if (token_route->experts % peers->world) return fail_arg("ep_push_dispatch: experts must divide evenly over the ranks");
    if (token_route->rows_bound >= (1ll << kRetRankShift)) return fail_arg("ep_push_dispatch: too many rows for the return-address encoding");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_EXCHANGE, stream);
    ep_push_dispatch_kernel<<<push_grid(token_route->rows_bound, blocks_per_sm), 256, 0, stream>>>(
        (const uint4*)src, row_bytes / 16, (const int*)token_route->tile_expert, (const int*)token_route->offsets,
        (const int*)token_route->counts, (const int*)token_route->meta, (const int*)dest_base,
        token_route->experts / peers->world, peers->rank, make_table(peers, write_return_addresses != 0));
    QMOE_LAUNCH_CHECK("ep_push_dispatch_kernel");
    return 0;
}

extern "C" int qmoe_ep_push_return(const qmoe_route_t* expert_route, uint64_t return_addresses, uint64_t src,
                                   const qmoe_ep_peers_t* peers, int32_t expert_begin, int32_t expert_end,
                                   int32_t blocks_per_sm, int32_t dtype, int64_t width, uint64_t stream_) {
    if (int rc = route_check(expert_route)) return rc;
    if (int rc = check_peers(peers, false)) return rc;
    if (!return_addresses || !src || (src & 15u)) return fail_arg("ep_push_return: null or misaligned buffer");
    if (expert_begin < 0 || expert_end > expert_route->experts || expert_begin > expert_end)
        return fail_arg("ep_push_return: expert range [%d, %d) is outside [0, %d)", expert_begin, expert_end, expert_route->experts);
    const long long row_bytes = width * (dtype == QMOE_BF16 ? 2 : 4);
    if (width <= 0 || row_bytes % 16) return fail_arg("ep_push_return: rows must be multiples of 16 bytes");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_EXCHANGE, stream);
    ep_push_return_kernel<<<push_grid(expert_route->rows_bound, blocks_per_sm), 256, 0, stream>>>(
        (const uint4*)src, row_bytes / 16, (const int*)expert_route->tile_expert, (const int*)expert_route->offsets,
        (const int*)expert_route->counts, (const int*)expert_route->meta, (const int*)return_addresses, expert_begin,
        expert_end, make_table(peers, false));
    QMOE_LAUNCH_CHECK("ep_push_return_kernel");
    return 0;
}

// ---------------------------------------------------------------------------------------------
// Fused producers: the kernels that create the rows write them straight into the destination GPU's
// buffer, so no separate exchange pass remains — the token-side permute and combine-backward scatter
// to the expert ranks, and the two row products of the expert FFN (down projection, dX) store their
// tiles at the rows' return addresses from the tensor-core epilogue.
// ---------------------------------------------------------------------------------------------
namespace qmoe {
namespace {

__device__ __forceinline__ uint4 ldg16_stream(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

struct SlotTarget {
    uint4* row;   // destination row on the owning rank
};

// x[t] -> the k expert-side rows of token t, wherever they live; records the return address of each
template <int KMAX>
__global__ void __launch_bounds__(256)
ep_permute_push_kernel(const uint4* __restrict__ x, long long row_vecs, const int* __restrict__ expert_index,
                       const int* __restrict__ dest_row, const int* __restrict__ offsets, const int* __restrict__ dest_base,
                       long long tokens, int k, int E_loc, int rank, int local_begin, int local_end, PeerTable peers) {
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    for (long long t = warp; t < tokens; t += nwarps) {
        uint4* target[KMAX];
        bool any = false;
#pragma unroll
        for (int s = 0; s < KMAX; ++s) {
            target[s] = nullptr;
            if (s < k) {
                const long long a = t * k + s;
                const int e = expert_index[a], r = dest_row[a];
                const int p = e / E_loc, local = e - p * E_loc;
                if (local < local_begin || local >= local_end) continue;  // this slot's expert travels with another call
                const long long dest = (long long)dest_base[e] + (r - offsets[e]);
                target[s] = peers.buffer[p] + dest * row_vecs;
                any = true;
                if (lane == 0) peers.ret[p][dest] = (rank << kRetRankShift) | r;
            }
        }
        if (!any) continue;
        const uint4* src = x + t * row_vecs;
        long long c = lane;
        for (; c + 32 < row_vecs; c += 64) {
            const uint4 v0 = ldg16_stream(src + c), v1 = ldg16_stream(src + c + 32);
#pragma unroll
            for (int s = 0; s < KMAX; ++s)
                if (target[s]) { target[s][c] = v0; target[s][c + 32] = v1; }
        }
        for (; c < row_vecs; c += 32) {
            const uint4 v0 = ldg16_stream(src + c);
#pragma unroll
            for (int s = 0; s < KMAX; ++s)
                if (target[s]) target[s][c] = v0;
        }
    }
    __threadfence_system();
}

// dY row of (t, s) = g[t] * w[t, s] -> its expert-side row; d_gate_weights[t, s] = <g[t], y_send[dest_row[t, s]]>
template <typename T, int KMAX>
__global__ void __launch_bounds__(256)
ep_combine_backward_push_kernel(const T* __restrict__ g, const T* __restrict__ y, const float* __restrict__ gate_w,
                                const int* __restrict__ expert_index, const int* __restrict__ dest_row,
                                const int* __restrict__ offsets, const int* __restrict__ dest_base, float* __restrict__ dw,
                                long long tokens, int k, long long width, int E_loc, int local_begin, int local_end,
                                PeerTable peers) {
    constexpr int N = Vec16<T>::N;
    const int lane = threadIdx.x & 31;
    const long long warp = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const long long nwarps = (long long)gridDim.x * (blockDim.x >> 5);
    const int chunks = (int)(width / N);
    for (long long t = warp; t < tokens; t += nwarps) {
        T* target[KMAX];
        long long local[KMAX];
        float w[KMAX], dot[KMAX];
        bool any = false;
#pragma unroll
        for (int s = 0; s < KMAX; ++s) {
            target[s] = nullptr; local[s] = 0; w[s] = 0.f; dot[s] = 0.f;
            if (s < k) {
                const long long a = t * k + s;
                const int e = expert_index[a], r = dest_row[a];
                const int owner = e / E_loc, slot = e - owner * E_loc;
                if (slot < local_begin || slot >= local_end) continue;  // this slot's expert travels with another call
                const long long dest = (long long)dest_base[e] + (r - offsets[e]);
                target[s] = (T*)peers.buffer[owner] + dest * width;
                local[s] = r;
                w[s] = gate_w[a];
                any = true;
            }
        }
        if (!any) continue;
        const T* gs = g + t * width;
        for (int c = lane; c < chunks; c += 32) {
            float fg[N];
            Vec16<T>::unpack(ldg16_stream(gs + (long long)c * N), fg);
            uint4 v[KMAX];
#pragma unroll
            for (int s = 0; s < KMAX; ++s)
                if (target[s]) v[s] = ldg16_stream(y + local[s] * width + (long long)c * N);
#pragma unroll
            for (int s = 0; s < KMAX; ++s)
                if (target[s]) {
                    float fy[N], o[N];
                    Vec16<T>::unpack(v[s], fy);
#pragma unroll
                    for (int i = 0; i < N; ++i) { dot[s] = fmaf(fg[i], fy[i], dot[s]); o[i] = fg[i] * w[s]; }
                    *reinterpret_cast<uint4*>(target[s] + (long long)c * N) = Vec16<T>::pack(o);
                }
        }
#pragma unroll
        for (int s = 0; s < KMAX; ++s)
            if (target[s]) {   // uniform over the warp: every lane holds the same targets
                const float total = warp_sum(dot[s]);
                if (lane == 0) dw[t * k + s] = total;
            }
    }
    __threadfence_system();
}

int check_push_rows(int dtype, long long width, std::initializer_list<uint64_t> ptrs) {
    if (dtype != QMOE_BF16 && dtype != QMOE_F32) return fail_arg("bad dtype %d", dtype);
    if (width <= 0 || (width * (dtype == QMOE_BF16 ? 2 : 4)) % 16) return fail_arg("rows must be multiples of 16 bytes");
    for (uint64_t p : ptrs)
        if (!p || (p & 15u)) return fail_arg("null or misaligned buffer");
    return 0;
}

int token_grid(long long tokens) {
    long long blocks = (tokens + 7) / 8;
    const long long cap = (long long)sm_count() * 8;
    return (int)(blocks > cap ? cap : (blocks < 1 ? 1 : blocks));
}

void fill_scatter(TcScatter& s, uint64_t ret, const qmoe_ep_peers_t* peers) {
    s.ret = (const int*)ret;
    for (int i = 0; i < 16; ++i) s.base[i] = i < peers->world ? peers->buffer[i] : 0;
}

}  // namespace
}  // namespace qmoe

extern "C" int qmoe_ep_permute_push(const qmoe_route_t* r, uint64_t dest_base, uint64_t x, const qmoe_ep_peers_t* peers,
                                    int32_t dtype, int64_t width, uint64_t stream) {
    return qmoe_ep_permute_push_range(r, dest_base, x, peers, 0, QMOE_MAX_EXPERTS, dtype, width, stream);
}

extern "C" int qmoe_ep_permute_push_range(const qmoe_route_t* r, uint64_t dest_base, uint64_t x, const qmoe_ep_peers_t* peers,
                                          int32_t local_begin, int32_t local_end, int32_t dtype, int64_t width,
                                          uint64_t stream_) {
    if (int rc = route_check(r)) return rc;
    if (local_begin < 0 || local_end < local_begin) return fail_arg("ep_permute_push: bad local expert range [%d, %d)", local_begin, local_end);
    if (int rc = check_peers(peers, true)) return rc;
    if (int rc = check_push_rows(dtype, width, {x, dest_base})) return rc;
    if (r->experts % peers->world) return fail_arg("ep_permute_push: experts must divide evenly over the ranks");
    if (r->rows_bound >= (1ll << kRetRankShift)) return fail_arg("ep_permute_push: too many rows for the return-address encoding");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_EXCHANGE, stream);
    const long long row_vecs = width * (dtype == QMOE_BF16 ? 2 : 4) / 16;
    const int E_loc = r->experts / peers->world, grid = token_grid(r->tokens);
    const PeerTable table = make_table(peers, true);
#define LAUNCH(K) ep_permute_push_kernel<K><<<grid, 256, 0, stream>>>((const uint4*)x, row_vecs, (const int*)r->expert_index, \
        (const int*)r->dest_row, (const int*)r->offsets, (const int*)dest_base, r->tokens, r->top_k, E_loc, peers->rank,      \
        local_begin, local_end, table)
    if (r->top_k <= 1) LAUNCH(1); else if (r->top_k <= 2) LAUNCH(2); else if (r->top_k <= 4) LAUNCH(4);
    else if (r->top_k <= 6) LAUNCH(6); else LAUNCH(8);
#undef LAUNCH
    QMOE_LAUNCH_CHECK("ep_permute_push_kernel");
    return 0;
}

extern "C" int qmoe_ep_combine_backward_push(const qmoe_route_t* r, uint64_t dest_base, uint64_t grad_out, uint64_t y_local,
                                             const qmoe_ep_peers_t* peers, uint64_t d_gate_weights, int32_t dtype,
                                             int64_t width, uint64_t stream) {
    return qmoe_ep_combine_backward_push_range(r, dest_base, grad_out, y_local, peers, d_gate_weights, 0, QMOE_MAX_EXPERTS,
                                               dtype, width, stream);
}

extern "C" int qmoe_ep_combine_backward_push_range(const qmoe_route_t* r, uint64_t dest_base, uint64_t grad_out,
                                                   uint64_t y_local, const qmoe_ep_peers_t* peers, uint64_t d_gate_weights,
                                                   int32_t local_begin, int32_t local_end, int32_t dtype, int64_t width,
                                                   uint64_t stream_) {
    if (int rc = route_check(r)) return rc;
    if (local_begin < 0 || local_end < local_begin) return fail_arg("ep_combine_backward_push: bad local expert range [%d, %d)", local_begin, local_end);
    if (int rc = check_peers(peers, false)) return rc;
    if (int rc = check_push_rows(dtype, width, {grad_out, y_local, dest_base})) return rc;
    if (!d_gate_weights) return fail_arg("ep_combine_backward_push: d_gate_weights is null");
    if (r->experts % peers->world) return fail_arg("ep_combine_backward_push: experts must divide evenly over the ranks");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_EXCHANGE, stream);
    const int E_loc = r->experts / peers->world, grid = token_grid(r->tokens);
    const PeerTable table = make_table(peers, false);
#define LAUNCH(T, K) ep_combine_backward_push_kernel<T, K><<<grid, 256, 0, stream>>>((const T*)grad_out, (const T*)y_local, \
        (const float*)r->gate_weights, (const int*)r->expert_index, (const int*)r->dest_row, (const int*)r->offsets,            \
        (const int*)dest_base, (float*)d_gate_weights, r->tokens, r->top_k, (long long)width, E_loc, local_begin, local_end, table)
#define BY_K(T) do { if (r->top_k <= 1) LAUNCH(T, 1); else if (r->top_k <= 2) LAUNCH(T, 2); else if (r->top_k <= 4) LAUNCH(T, 4); \
                     else if (r->top_k <= 6) LAUNCH(T, 6); else LAUNCH(T, 8); } while (0)
    if (dtype == QMOE_BF16) BY_K(__nv_bfloat16); else BY_K(float);
#undef BY_K
#undef LAUNCH
    QMOE_LAUNCH_CHECK("ep_combine_backward_push_kernel");
    return 0;
}

extern "C" int qmoe_ep_expert_down_push(const qmoe_route_t* expert_route, const qmoe_experts_t* ex, uint64_t h,
                                        uint64_t return_addresses, const qmoe_ep_peers_t* peers, uint64_t stream_) {
    if (int rc = route_check(expert_route)) return rc;
    if (int rc = check_peers(peers, false)) return rc;
    if (!ex || !h || !return_addresses || !ex->w_down) return fail_arg("ep_expert_down_push: null argument");
    if (ex->dtype != QMOE_BF16 || !tcgen05_shape_ok(ex->width, ex->hidden) || ex->engine == QMOE_ENGINE_SIMT) {
        set_error("ep_expert_down_push needs the tensor-core engine (bf16 activations, widths multiples of 8)");
        return QMOE_ERR_UNSUPPORTED;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_EXPERT_GEMM, stream);
    TcScatter scatter;
    fill_scatter(scatter, return_addresses, peers);
    return tc_rows_nt(expert_route, ex->experts, h, ex->w_down, peers->buffer[peers->rank], ex->hidden, ex->width, stream, &scatter);
}

extern "C" int qmoe_ep_expert_dx_push(const qmoe_route_t* expert_route, const qmoe_experts_t* ex, uint64_t d_g, uint64_t d_u,
                                      uint64_t return_addresses, const qmoe_ep_peers_t* peers, uint64_t stream_) {
    if (int rc = route_check(expert_route)) return rc;
    if (int rc = check_peers(peers, false)) return rc;
    if (!ex || !d_g || !d_u || !return_addresses || !ex->w_gate || !ex->w_up) return fail_arg("ep_expert_dx_push: null argument");
    if (ex->dtype != QMOE_BF16 || !tcgen05_shape_ok(ex->width, ex->hidden) || ex->engine == QMOE_ENGINE_SIMT) {
        set_error("ep_expert_dx_push needs the tensor-core engine (bf16 activations, widths multiples of 8)");
        return QMOE_ERR_UNSUPPORTED;
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_EXPERT_GEMM, stream);
    TcScatter scatter;
    fill_scatter(scatter, return_addresses, peers);
    return tc_rows_nn(expert_route, ex->experts, d_g, ex->w_gate, d_u, ex->w_up, peers->buffer[peers->rank], ex->hidden,
                      ex->width, stream, &scatter);
}

// ---------------------------------------------------------------------------------------------
// Flag barrier over peer memory: every rank stores the barrier's sequence number into its slot of
// every rank's flag array, then waits until all slots of its own array carry that number.  Each
// GPU runs its own copy of the kernel; the wait is bounded (ten seconds unless set otherwise), after which the
// kernel records a code in the status word and returns, so a missing rank shows up as a status on
// the others instead of a hang.  Sequence numbers only grow, so the flags never need resetting.
// ---------------------------------------------------------------------------------------------
namespace qmoe {
namespace {

constexpr int kStatusBarrierTimeout = 201;
// How long a rank waits for the others before it gives up.  Seconds of skew between the hosts of a training
// job are normal (a checkpoint write, a data-loader stall, logging on one rank), so the default is generous;
// qmoe_ep_set_barrier_timeout_ms changes it (the failure-detection test asks for a fraction of a second).
std::atomic<long long> g_barrier_wait_ns{10ll * 1000 * 1000 * 1000};

struct FlagTable {
    int* flags[kMaxPeers];
};

__device__ __forceinline__ unsigned long long barrier_clock_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Optionally also publishes this rank's 2E statistics words into slot `rank` of every rank's table
// (the all-gather of the routing counts), before the flags are raised.
__global__ void __launch_bounds__(512)
ep_flag_barrier_kernel(FlagTable table, int rank, int world, int sequence, int* status, const int* stats_local,
                       int stats_words, FlagTable stats_tables, unsigned long long wait_ns) {
    if (stats_local) {
        for (int i = threadIdx.x; i < stats_words * world; i += blockDim.x) {
            const int p = i / stats_words, j = i - p * stats_words;
            stats_tables.flags[p][(long long)rank * stats_words + j] = stats_local[j];
        }
        __threadfence_system();
        __syncthreads();
    }
    const int p = threadIdx.x;
    if (p >= world) return;
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(table.flags[p] + rank), "r"(sequence) : "memory");
    const int* mine = table.flags[rank] + p;
    const unsigned long long start = barrier_clock_ns();
    for (unsigned spin = 0;; ++spin) {
        int seen;
        asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
        if (seen - sequence >= 0) break;
        if ((spin & 255u) == 255u && barrier_clock_ns() - start > wait_ns) {
            atomicExch(status, kStatusBarrierTimeout);
            break;
        }
    }
}

}  // namespace
}  // namespace qmoe

extern "C" int qmoe_ep_flag_barrier(const qmoe_ep_peers_t* flags, int32_t sequence, uint64_t stats_local,
                                    int32_t stats_words, const qmoe_ep_peers_t* stats_tables, uint64_t stream_) {
    if (!flags) return fail_arg("ep_flag_barrier: flags is null");
    if (flags->world <= 0 || flags->world > kMaxPeers || flags->rank < 0 || flags->rank >= flags->world)
        return fail_arg("ep_flag_barrier: bad world / rank");
    if (sequence <= 0) return fail_arg("ep_flag_barrier: the sequence number must be positive and growing");
    if (stats_local && (!stats_tables || stats_words <= 0)) return fail_arg("ep_flag_barrier: statistics tables are missing");
    FlagTable table = {}, stats = {};
    for (int p = 0; p < flags->world; ++p) {
        if (!flags->buffer[p]) return fail_arg("ep_flag_barrier: flag array of rank %d is null", p);
        table.flags[p] = (int*)flags->buffer[p];
        if (stats_local) {
            if (!stats_tables->buffer[p]) return fail_arg("ep_flag_barrier: statistics table of rank %d is null", p);
            stats.flags[p] = (int*)stats_tables->buffer[p];
        }
    }
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_BARRIER, stream);
    ep_flag_barrier_kernel<<<1, 512, 0, stream>>>(table, flags->rank, flags->world, sequence, device_status_address(),
                                                  (const int*)stats_local, stats_words, stats,
                                                  (unsigned long long)g_barrier_wait_ns.load());
    QMOE_LAUNCH_CHECK("ep_flag_barrier_kernel");
    return 0;
}

extern "C" int qmoe_ep_set_barrier_timeout_ms(int64_t milliseconds) {
    if (milliseconds <= 0 || milliseconds > 600000) return fail_arg("ep_set_barrier_timeout_ms: need 1 .. 600000 ms");
    g_barrier_wait_ns.store((long long)milliseconds * 1000000ll);
    return 0;
}

// the local half of qmoe_ep_gather_stats: pack {counts, column sums} without the NCCL all-gather
extern "C" int qmoe_ep_pack_stats(const qmoe_route_t* r, uint64_t stats_local, uint64_t stream_) {
    if (int rc = route_check(r)) return rc;
    if (!stats_local) return fail_arg("ep_pack_stats: null buffer");
    if (!r->block_colsum) return fail_arg("ep_pack_stats: route.block_colsum is null (a route filled by qmoe_route_static keeps its column sums inside the library)");
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_OTHER, stream);
    ep_stats_kernel<<<1, kMaxExperts, 0, stream>>>((const int*)r->counts, (const float*)r->block_colsum,
                                                    (int)qmoe_route_blocks(r->tokens), r->experts, (int*)stats_local);
    QMOE_LAUNCH_CHECK("ep_stats_kernel");
    return 0;
}
