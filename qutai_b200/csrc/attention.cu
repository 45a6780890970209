// Causal self-attention with grouped key/value heads, head width 64, bf16 in and out, on the tcgen05 tensor cores:
//     out[b, t, h, :] = sum_{s <= t} softmax_s(q[b, t, h, :] . k[b, s, g(h), :] / 8) v[b, s, g(h), :],  g(h) = h / (heads / kv_heads)
// forward (with the log-sum-exp of every row kept for the backward) and backward (dq, dk, dv).
// Upstream: `attention` src/qutai/lm/layers.py:119-130, kernels lm_attention_bf16_d64 / _dq / _dkv
// src/qutai/backends/cuda/lm.cu:91-285 (wmma), CPU statement src/qutai/backends/cpu_lm.py:141-201.  Like those kernels
// this never writes the time x time scores: keys and values stream through shared memory in blocks of 128 positions.
//
// One CTA per (sequence, head, block of 128 query positions); 6 warps: warp 0 asks TMA for the tiles (3-D tensor maps
// [batch][time][heads * 64], so positions past the end of a sequence arrive as zeros and no tile reaches into the next
// sequence), warp 1 issues the MMAs (one thread), warps 2-5 own one query row per thread (the TMEM lane of that row).
//   forward, per key block:  S = Q K^T (TMEM) -> rows: max, exp2, sum; P (bf16) into shared memory in the K-major
//   operand layout -> O_j = P V (TMEM) -> rows: O = O * alpha + O_j in registers.
//   backward for dq, per key block:  S = Q K^T and dP = dO V^T (TMEM) -> rows: P = exp(S / 8 - lse),
//   dS = P (dP - delta) / 8 (bf16, shared memory) -> dQ += dS K (TMEM, accumulated over the key blocks).
//   backward for dk, dv, one CTA per (sequence, key/value head, key block), over the query heads of the group and
//   the query blocks at or after it:  S, dP as above -> P and dS (shared memory) -> dV += P^T dO, dK += dS^T Q
//   (TMEM; the K-major tile of P read as an MN-major operand is P^T, no transposed copy).
// Every wait is bounded; on expiry the CTA records a code in the library's status word and leaves.
#include "common.cuh"
#include "tc_ptx.cuh"

namespace qmoe {
namespace {

constexpr int D = 64;                 // head width
constexpr int BLOCK = 128;            // query rows of a CTA = key positions of a block
constexpr int TILE_BYTES = BLOCK * D * 2;          // 16 KiB: 128 rows x 128 bytes
constexpr int SLAB_BYTES = BLOCK * 128;            // one 64-column half of a 128 x 128 bf16 operand tile
constexpr int THREADS = 192;              // forward: TMA warp, MMA warp, four row warps
// The backward kernels have no reduction along a row (lse and delta are known), so the columns of a block are split
// between several warps per 32 rows: one warp per scheduler cannot hide its own arithmetic latency (measured: 4900 of
// the 7300 cycles of a dk/dv iteration were the four row warps' work).
constexpr int DQ_PARTS = 2, DKV_PARTS = 4;
constexpr int DQ_THREADS = 64 + 128 * DQ_PARTS, DKV_THREADS = 64 + 128 * DKV_PARTS;
constexpr float LOG2E = 1.4426950408889634f;
enum { STATUS_ATTENTION_WAIT = 301 };

struct alignas(64) AttentionParams {
    CUtensorMap map_q, map_k, map_v, map_do;     // 3-D [batch][time][heads * 64] bf16, boxes of 64 x 128 x 1
    CUtensorMap map_k2, map_v2;                  // the same tensors in boxes of 64 x 64 x 1 (dq kernel with key blocks of 64)
    const __nv_bfloat16* out_in;  // backward: the forward's output
    const __nv_bfloat16* grad_out;
    __nv_bfloat16* out;           // forward: out; backward for dq: dq; backward for dk, dv: dk
    __nv_bfloat16* out2;          // backward for dk, dv: dv
    float* lse;                   // [batch * time * heads]
    float* delta;                 // [batch * time * heads]  sum_j grad_out * out of every row
    int* status;
    int batch, time, heads, kv_heads;
};

__device__ __forceinline__ void tma_load_3d(const CUtensorMap* map, uint32_t dst, uint32_t bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ uint32_t pack2(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}
__device__ __forceinline__ float exp2_fast(float x) {
    float y;
    asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
// 32 consecutive values of this thread's row (columns [32 c, 32 c + 32) of a 128-column bf16 operand tile made of two
// 64-column slabs) into shared memory in the K-major layout the MMA reads: 128-byte rows, 16-byte piece j of row r at
// j ^ (r & 7)
__device__ __forceinline__ void store_row32(uint32_t tile, int row, int c, const uint32_t* packed16) {
    const uint32_t slab = tile + (uint32_t)(c >> 1) * SLAB_BYTES + (uint32_t)row * 128u;
    const uint32_t twist = (uint32_t)row & 7u;
#pragma unroll
    for (int piece = 0; piece < 4; ++piece) {
        const uint32_t at = (((uint32_t)(c & 1) * 4u + (uint32_t)piece) ^ twist) * 16u;
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(slab + at), "r"(packed16[4 * piece]), "r"(packed16[4 * piece + 1]),
                     "r"(packed16[4 * piece + 2]), "r"(packed16[4 * piece + 3]) : "memory");
    }
}

struct Wait {   // bounded waits of one thread; the first that runs out marks the CTA
    volatile int* abort_flag;
    int* status;
    __device__ __forceinline__ bool operator()(uint32_t bar, uint32_t parity) const {
        if (mbar_wait(bar, parity, abort_flag)) return true;
        if (!*abort_flag) { *abort_flag = 1; atomicExch(status, STATUS_ATTENTION_WAIT); }
        return false;
    }
};

// a CTA that gave up leaves its copies and MMAs in flight a bounded time to land before its shared memory and TMEM go away
__device__ __forceinline__ void linger_after_abort(const volatile int* abort_flag) {
    if (!*abort_flag) return;
    const unsigned long long start = global_ns();
    while (global_ns() - start < 2000000ull) __nanosleep(1000);
}

// ------------------------------------------------------------------------------------------------
// forward
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS)
attention_forward_kernel(const __grid_constant__ AttentionParams p) {
    // No static shared memory and a 1 KiB-aligned dynamic block: 112 KiB of tiles + the barriers and two words fit
    // twice into an SM, and the second resident CTA is what overlaps one CTA's row work with another's MMAs.
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blocks = (p.time + BLOCK - 1) / BLOCK;
    // heaviest query blocks first: the last block of a sequence has the most key blocks to walk
    const int i = blocks - 1 - (int)(blockIdx.x % blocks);
    const int h = (int)(blockIdx.x / blocks) % p.heads, b = (int)(blockIdx.x / blocks) / p.heads;
    const int g = h / (p.heads / p.kv_heads);
    const int n = i + 1;                       // key blocks 0 .. i
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t q_tile = base, k_tile = base + TILE_BYTES, v_tile = k_tile + 2 * TILE_BYTES, p_tile = v_tile + 2 * TILE_BYTES;
    const uint32_t bars = p_tile + 2 * SLAB_BYTES;
    enum { Q_FULL = 0, KV_FULL = 1, KV_EMPTY = 3, S_FULL = 5, P_FULL = 6, O_FULL = 7, O_TAKEN = 8, BARS = 9 };
    auto bar = [&](int which) { return bars + 8u * which; };
    uint32_t& s_tmem_base = *reinterpret_cast<uint32_t*>(smem_raw + 5 * TILE_BYTES + 2 * SLAB_BYTES + 8 * BARS);
    volatile int& s_abort = *reinterpret_cast<volatile int*>(smem_raw + 5 * TILE_BYTES + 2 * SLAB_BYTES + 8 * BARS + 4);
    if (base & 1023u) {   // the operand tiles need the alignment the declaration asks for
        if (threadIdx.x == 0) atomicExch(p.status, STATUS_ATTENTION_WAIT + 1);
        return;
    }
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int w = 0; w < BARS; ++w) mbar_init(bar(w), (w == P_FULL || w == O_TAKEN) ? 4 : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_map(&p.map_q); prefetch_map(&p.map_k); prefetch_map(&p.map_v);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(256) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;
    const uint32_t tmem_s = tmem, tmem_o = tmem + 128;
    const Wait wait{&s_abort, p.status};

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(bar(Q_FULL), TILE_BYTES);
            tma_load_3d(&p.map_q, q_tile, bar(Q_FULL), h * D, i * BLOCK, b);
            for (int j = 0; j < n && !s_abort; ++j) {
                const int st = j & 1;
                if (!wait(bar(KV_EMPTY + st), ((uint32_t)(j >> 1) & 1u) ^ 1u)) break;
                mbar_expect_tx(bar(KV_FULL + st), 2 * TILE_BYTES);
                tma_load_3d(&p.map_k, k_tile + st * TILE_BYTES, bar(KV_FULL + st), g * D, j * BLOCK, b);
                tma_load_3d(&p.map_v, v_tile + st * TILE_BYTES, bar(KV_FULL + st), g * D, j * BLOCK, b);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc<false, false, 128>(128), idesc_o = make_idesc<false, true, 128>(D);
            bool ok = wait(bar(Q_FULL), 0);
            for (int j = 0; ok && j < n; ++j) {
                const int st = j & 1;
                ok = wait(bar(KV_FULL + st), (uint32_t)(j >> 1) & 1u);
                if (!ok) break;
                tc_fence_after();
                // S = Q K^T: both K-major, contraction over the 64 columns (the rows that read S of the block
                // before have all arrived on P_FULL, which was waited for before that block's P V)
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)
                    umma_bf16(tmem_s, make_desc(q_tile + kk * 32, 16, 1024), make_desc(k_tile + st * TILE_BYTES + kk * 32, 16, 1024), idesc_s, kk ? 1u : 0u);
                umma_commit(bar(S_FULL));
                ok = wait(bar(P_FULL), (uint32_t)j & 1u);
                if (ok && j > 0) ok = wait(bar(O_TAKEN), (uint32_t)(j - 1) & 1u);
                if (!ok) break;
                tc_fence_after();
                // O_j = P V: P K-major (two 64-column slabs), V as it lies in memory (rows = key positions) is the
                // MN-major operand: 16 positions every 2 KiB
#pragma unroll
                for (int kk = 0; kk < BLOCK / 16; ++kk)
                    umma_bf16(tmem_o, make_desc(p_tile + (kk >> 2) * SLAB_BYTES + (kk & 3) * 32, 16, 1024),
                              make_desc(v_tile + st * TILE_BYTES + kk * 2048, 8192, 1024), idesc_o, kk ? 1u : 0u);
                umma_commit(bar(O_FULL));
                umma_commit(bar(KV_EMPTY + st));
            }
            // the last commit has arrived before this CTA's shared memory can go to another one
            if (ok) wait(bar(KV_EMPTY + ((n - 1) & 1)), (uint32_t)((n - 1) >> 1) & 1u);
        }
    } else {
        const int quad = warp & 3, row = quad * 32 + lane;
        const int tq = i * BLOCK + row;                      // this thread's query position
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const float scale2 = 0.125f * LOG2E;                 // 1 / sqrt(64), in the exponent of 2
        float m = -INFINITY, l = 0.f, o[D];
#pragma unroll
        for (int c = 0; c < D; ++c) o[c] = 0.f;
        bool ok = true;
        for (int j = 0; ok && j < n; ++j) {
            ok = wait(bar(S_FULL), (uint32_t)j & 1u);
            if (!ok) break;
            tc_fence_after();
            const bool diagonal = j == i;
            float peak = m;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_s + lane_base + c * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e)
                    if (!diagonal || c * 32 + e <= row) peak = fmaxf(peak, __uint_as_float(r[e]));
            }
            const float alpha = exp2_fast((m - peak) * scale2);   // 0 in the first block (m = -inf, peak finite: column 0 is never masked)
            float total = 0.f;
#pragma unroll 1
            for (int c = 0; c < 4; ++c) {
                uint32_t r[32], packed[16];
                tmem_ld32(tmem_s + lane_base + c * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float p0 = exp2_fast((__uint_as_float(r[e]) - peak) * scale2), p1 = exp2_fast((__uint_as_float(r[e + 1]) - peak) * scale2);
                    if (diagonal && c * 32 + e > row) p0 = 0.f;
                    if (diagonal && c * 32 + e + 1 > row) p1 = 0.f;
                    total += p0 + p1;
                    packed[e >> 1] = pack2(p0, p1);
                }
                store_row32(p_tile, row, c, packed);
            }
            l = l * alpha + total;
            m = peak;
            fence_async_shared();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(P_FULL));
            ok = wait(bar(O_FULL), (uint32_t)j & 1u);
            if (!ok) break;
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t r[32];
                tmem_ld32(tmem_o + lane_base + c * 32, r);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; ++e) o[c * 32 + e] = o[c * 32 + e] * alpha + __uint_as_float(r[e]);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(O_TAKEN));
        }
        if (ok && tq < p.time) {
            const float inverse = 1.f / l;
            const long long at = ((long long)b * p.time + tq) * p.heads + h;
            uint4* dst = reinterpret_cast<uint4*>(p.out + at * D);
#pragma unroll
            for (int c = 0; c < D / 8; ++c)
                dst[c] = make_uint4(pack2(o[8 * c] * inverse, o[8 * c + 1] * inverse), pack2(o[8 * c + 2] * inverse, o[8 * c + 3] * inverse),
                                    pack2(o[8 * c + 4] * inverse, o[8 * c + 5] * inverse), pack2(o[8 * c + 6] * inverse, o[8 * c + 7] * inverse));
            p.lse[at] = m * 0.125f + __logf(l);
        }
    }
    linger_after_abort(&s_abort);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(256) : "memory");
    }
}


// ------------------------------------------------------------------------------------------------
// backward, part 1: dq (and delta), one CTA per (sequence, head, query block); key blocks of KV positions.  With
// KV = 64 a CTA needs 192 TMEM columns and 80 KiB, so two are resident per SM and overlap each other's chains.
// ------------------------------------------------------------------------------------------------
template <int KV>
__global__ void __launch_bounds__(DQ_THREADS)
attention_dq_kernel(const __grid_constant__ AttentionParams p) {
    constexpr int KV_TILE = KV * 128, SLABS = KV / 64, TMEM_COLUMNS = KV == 64 ? 256 : 512;
    constexpr int TILES = 2 * TILE_BYTES + 4 * KV_TILE + SLABS * SLAB_BYTES;
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blocks = (p.time + BLOCK - 1) / BLOCK;
    const int i = blocks - 1 - (int)(blockIdx.x % blocks);
    const int h = (int)(blockIdx.x / blocks) % p.heads, b = (int)(blockIdx.x / blocks) / p.heads;
    const int g = h / (p.heads / p.kv_heads);
    const int n = (i + 1) * (BLOCK / KV);      // key blocks that hold a position <= the last query of this block
    const uint32_t base = smem_u32(smem_raw);
    const uint32_t q_tile = base, do_tile = base + TILE_BYTES, k_tile = do_tile + TILE_BYTES, v_tile = k_tile + 2 * KV_TILE,
                   ds_tile = v_tile + 2 * KV_TILE;
    const uint32_t bars = ds_tile + SLABS * SLAB_BYTES;
    enum { Q_FULL = 0, KV_FULL = 1, KV_EMPTY = 3, SP_FULL = 5, DS_FULL = 6, DQ_DONE = 7, BARS = 8 };
    auto bar = [&](int which) { return bars + 8u * which; };
    uint32_t& s_tmem_base = *reinterpret_cast<uint32_t*>(smem_raw + TILES + 8 * BARS);
    volatile int& s_abort = *reinterpret_cast<volatile int*>(smem_raw + TILES + 8 * BARS + 4);
    if (base & 1023u) {
        if (threadIdx.x == 0) atomicExch(p.status, STATUS_ATTENTION_WAIT + 1);
        return;
    }
    const CUtensorMap* map_k = KV == 64 ? &p.map_k2 : &p.map_k;
    const CUtensorMap* map_v = KV == 64 ? &p.map_v2 : &p.map_v;
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int w = 0; w < BARS; ++w) mbar_init(bar(w), w == DS_FULL ? 4 * DQ_PARTS : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_map(&p.map_q); prefetch_map(map_k); prefetch_map(map_v); prefetch_map(&p.map_do);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(TMEM_COLUMNS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;
    const uint32_t tmem_s = tmem, tmem_dp = tmem + KV, tmem_dq = tmem + 2 * KV;
    const Wait wait{&s_abort, p.status};

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(bar(Q_FULL), 2 * TILE_BYTES);
            tma_load_3d(&p.map_q, q_tile, bar(Q_FULL), h * D, i * BLOCK, b);
            tma_load_3d(&p.map_do, do_tile, bar(Q_FULL), h * D, i * BLOCK, b);
            for (int j = 0; j < n && !s_abort; ++j) {
                const int st = j & 1;
                if (!wait(bar(KV_EMPTY + st), ((uint32_t)(j >> 1) & 1u) ^ 1u)) break;
                mbar_expect_tx(bar(KV_FULL + st), 2 * KV_TILE);
                tma_load_3d(map_k, k_tile + st * KV_TILE, bar(KV_FULL + st), g * D, j * KV, b);
                tma_load_3d(map_v, v_tile + st * KV_TILE, bar(KV_FULL + st), g * D, j * KV, b);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc<false, false, 128>(KV), idesc_dq = make_idesc<false, true, 128>(D);
            bool ok = wait(bar(Q_FULL), 0);
            for (int j = 0; ok && j < n; ++j) {
                const int st = j & 1;
                ok = wait(bar(KV_FULL + st), (uint32_t)(j >> 1) & 1u);
                if (!ok) break;
                tc_fence_after();
                // S = Q K^T and dP = dO V^T (the rows that read both of the block before have arrived on DS_FULL)
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)
                    umma_bf16(tmem_s, make_desc(q_tile + kk * 32, 16, 1024), make_desc(k_tile + st * KV_TILE + kk * 32, 16, 1024), idesc_s, kk ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)
                    umma_bf16(tmem_dp, make_desc(do_tile + kk * 32, 16, 1024), make_desc(v_tile + st * KV_TILE + kk * 32, 16, 1024), idesc_s, kk ? 1u : 0u);
                umma_commit(bar(SP_FULL));
                ok = wait(bar(DS_FULL), (uint32_t)j & 1u);
                if (!ok) break;
                tc_fence_after();
                // dQ += dS K: dS K-major (slabs of 64 key positions), the K tile read as the MN-major operand (rows = key positions)
#pragma unroll
                for (int kk = 0; kk < KV / 16; ++kk)
                    umma_bf16(tmem_dq, make_desc(ds_tile + (kk >> 2) * SLAB_BYTES + (kk & 3) * 32, 16, 1024),
                              make_desc(k_tile + st * KV_TILE + kk * 2048, 8192, 1024), idesc_dq, (j | kk) ? 1u : 0u);
                umma_commit(bar(DQ_DONE));          // dS may be overwritten, and after the last block dQ is complete
                umma_commit(bar(KV_EMPTY + st));
            }
            if (ok) wait(bar(KV_EMPTY + ((n - 1) & 1)), (uint32_t)((n - 1) >> 1) & 1u);   // the last commit has arrived
        }
    } else {
        const int quad = warp & 3, row = quad * 32 + lane, part = (warp - 2) >> 2;     // part: which columns of a block
        constexpr int CHUNKS = KV / 32 / DQ_PARTS;
        static_assert(CHUNKS >= 1, "a key block has fewer 32-column chunks than there are row warps per 32 rows");
        const int tq = i * BLOCK + row;
        const bool live = tq < p.time;
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const long long at = ((long long)b * p.time + (live ? tq : 0)) * p.heads + h;
        // delta = sum_j grad_out * out of this row (kept for the dk, dv kernel), lse of this row
        float delta = 0.f, lse2 = 0.f;
        if (live) {
            const uint4* go = reinterpret_cast<const uint4*>(p.grad_out + at * D);
            const uint4* oo = reinterpret_cast<const uint4*>(p.out_in + at * D);
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                const uint4 a = go[c], o = oo[c];
                const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, ow[4] = {o.x, o.y, o.z, o.w};
#pragma unroll
                for (int e = 0; e < 4; ++e)
                    delta += __uint_as_float(aw[e] << 16) * __uint_as_float(ow[e] << 16) +
                             __uint_as_float(aw[e] & 0xffff0000u) * __uint_as_float(ow[e] & 0xffff0000u);
            }
            if (part == 0) p.delta[at] = delta;
            lse2 = p.lse[at] * LOG2E;
        }
        const float scale2 = 0.125f * LOG2E;
        bool ok = true;
        for (int j = 0; ok && j < n; ++j) {
            ok = wait(bar(SP_FULL), (uint32_t)j & 1u);
            if (ok && j > 0) ok = wait(bar(DQ_DONE), (uint32_t)(j - 1) & 1u);     // the MMAs that read dS of the block before are done
            if (!ok) break;
            tc_fence_after();
            const int first = j * KV;                              // key position of this block's column 0
            const bool masked = first + KV - 1 > i * BLOCK;        // the block reaches past the first query of this CTA
#pragma unroll 1
            for (int c = part * CHUNKS; c < (part + 1) * CHUNKS; ++c) {
                uint32_t rs[32], rp[32], packed[16];
                tmem_ld32(tmem_s + lane_base + c * 32, rs);
                tmem_ld32(tmem_dp + lane_base + c * 32, rp);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float d0 = 0.f, d1 = 0.f;
                    if (live && !(masked && first + c * 32 + e > tq))
                        d0 = exp2_fast(__uint_as_float(rs[e]) * scale2 - lse2) * (__uint_as_float(rp[e]) - delta) * 0.125f;
                    if (live && !(masked && first + c * 32 + e + 1 > tq))
                        d1 = exp2_fast(__uint_as_float(rs[e + 1]) * scale2 - lse2) * (__uint_as_float(rp[e + 1]) - delta) * 0.125f;
                    packed[e >> 1] = pack2(d0, d1);
                }
                store_row32(ds_tile, row, c, packed);
            }
            fence_async_shared();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(DS_FULL));
        }
        if (ok) ok = wait(bar(DQ_DONE), (uint32_t)(n - 1) & 1u);
        if (ok) {
            tc_fence_after();
            uint4* dst = reinterpret_cast<uint4*>(p.out + at * D);
#pragma unroll
            for (int c = part; c < 2; c += DQ_PARTS) {
                uint32_t r[32];
                tmem_ld32(tmem_dq + lane_base + c * 32, r);
                tmem_ld_wait();
                if (live) {
#pragma unroll
                    for (int e = 0; e < 4; ++e)
                        dst[c * 4 + e] = make_uint4(pack2(__uint_as_float(r[8 * e]), __uint_as_float(r[8 * e + 1])),
                                                    pack2(__uint_as_float(r[8 * e + 2]), __uint_as_float(r[8 * e + 3])),
                                                    pack2(__uint_as_float(r[8 * e + 4]), __uint_as_float(r[8 * e + 5])),
                                                    pack2(__uint_as_float(r[8 * e + 6]), __uint_as_float(r[8 * e + 7])));
                }
            }
        }
    }
    linger_after_abort(&s_abort);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(TMEM_COLUMNS) : "memory");
    }
}

// ------------------------------------------------------------------------------------------------
// backward, part 2: dk and dv, one CTA per (sequence, key/value head, key block)
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(DKV_THREADS)
attention_dkv_kernel(const __grid_constant__ AttentionParams p) {
    extern __shared__ uint8_t smem_raw[];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int blocks = (p.time + BLOCK - 1) / BLOCK;
    const int j = (int)(blockIdx.x % blocks);                  // the first key block has the most query blocks to walk
    const int g = (int)(blockIdx.x / blocks) % p.kv_heads, b = (int)(blockIdx.x / blocks) / p.kv_heads;
    const int group = p.heads / p.kv_heads;
    const int per_head = blocks - j;                           // query blocks j .. blocks - 1
    const int n = group * per_head;                            // iterations: head of the group (outer), query block (inner)
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t k_tile = base, v_tile = base + TILE_BYTES, q_tile = v_tile + TILE_BYTES, do_tile = q_tile + 2 * TILE_BYTES,
                   p_tile = do_tile + 2 * TILE_BYTES, ds_tile = p_tile + 2 * SLAB_BYTES;
    const uint32_t bars = ds_tile + 2 * SLAB_BYTES;
    enum { KV_FULL = 0, Q_FULL = 1, Q_EMPTY = 3, SP_FULL = 5, PDS_FULL = 6, ACC_DONE = 7, BARS = 8 };
    auto bar = [&](int which) { return bars + 8u * which; };
    if (threadIdx.x == 0) {
        s_abort = 0;
        for (int w = 0; w < BARS; ++w) mbar_init(bar(w), w == PDS_FULL ? 4 * DKV_PARTS : 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_map(&p.map_q); prefetch_map(&p.map_k); prefetch_map(&p.map_v); prefetch_map(&p.map_do);
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(512) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;
    const uint32_t tmem_s = tmem, tmem_dp = tmem + 128, tmem_dv = tmem + 256, tmem_dk = tmem + 320;
    const Wait wait{&s_abort, p.status};

    if (warp == 0) {
        if (lane == 0) {
            mbar_expect_tx(bar(KV_FULL), 2 * TILE_BYTES);
            tma_load_3d(&p.map_k, k_tile, bar(KV_FULL), g * D, j * BLOCK, b);
            tma_load_3d(&p.map_v, v_tile, bar(KV_FULL), g * D, j * BLOCK, b);
            for (int it = 0; it < n && !s_abort; ++it) {
                const int st = it & 1, h = g * group + it / per_head, i = j + it % per_head;
                if (!wait(bar(Q_EMPTY + st), ((uint32_t)(it >> 1) & 1u) ^ 1u)) break;
                mbar_expect_tx(bar(Q_FULL + st), 2 * TILE_BYTES);
                tma_load_3d(&p.map_q, q_tile + st * TILE_BYTES, bar(Q_FULL + st), h * D, i * BLOCK, b);
                tma_load_3d(&p.map_do, do_tile + st * TILE_BYTES, bar(Q_FULL + st), h * D, i * BLOCK, b);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc_s = make_idesc<false, false, 128>(128), idesc_t = make_idesc<true, true, 128>(D);
            bool ok = wait(bar(KV_FULL), 0);
            for (int it = 0; ok && it < n; ++it) {
                const int st = it & 1;
                ok = wait(bar(Q_FULL + st), (uint32_t)(it >> 1) & 1u);
                if (!ok) break;
                tc_fence_after();
                // S = Q K^T and dP = dO V^T, rows = query positions
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)
                    umma_bf16(tmem_s, make_desc(q_tile + st * TILE_BYTES + kk * 32, 16, 1024), make_desc(k_tile + kk * 32, 16, 1024), idesc_s, kk ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < D / 16; ++kk)
                    umma_bf16(tmem_dp, make_desc(do_tile + st * TILE_BYTES + kk * 32, 16, 1024), make_desc(v_tile + kk * 32, 16, 1024), idesc_s, kk ? 1u : 0u);
                umma_commit(bar(SP_FULL));
                ok = wait(bar(PDS_FULL), (uint32_t)it & 1u);
                if (!ok) break;
                tc_fence_after();
                // dV += P^T dO and dK += dS^T Q: the K-major tiles of P and dS (rows = query positions, two slabs of 64 key
                // positions) read as MN-major operands are their transposes; dO and Q read as MN-major operands
                // (rows = query positions = the contraction)
#pragma unroll
                for (int kk = 0; kk < BLOCK / 16; ++kk)
                    umma_bf16(tmem_dv, make_desc(p_tile + kk * 2048, SLAB_BYTES, 1024), make_desc(do_tile + st * TILE_BYTES + kk * 2048, 8192, 1024),
                              idesc_t, (it | kk) ? 1u : 0u);
#pragma unroll
                for (int kk = 0; kk < BLOCK / 16; ++kk)
                    umma_bf16(tmem_dk, make_desc(ds_tile + kk * 2048, SLAB_BYTES, 1024), make_desc(q_tile + st * TILE_BYTES + kk * 2048, 8192, 1024),
                              idesc_t, (it | kk) ? 1u : 0u);
                umma_commit(bar(ACC_DONE));        // P and dS may be overwritten; after the last iteration dV and dK are complete
                umma_commit(bar(Q_EMPTY + st));
            }
            if (ok) wait(bar(Q_EMPTY + ((n - 1) & 1)), (uint32_t)((n - 1) >> 1) & 1u);    // the last commit has arrived
        }
    } else {
        const int quad = warp & 3, row = quad * 32 + lane, part = (warp - 2) >> 2;     // part: which 32 columns of a block
        static_assert(DKV_PARTS == 4, "one 32-column chunk of S and dP, and one of the four chunks of dV and dK, per row warp");
        const uint32_t lane_base = (uint32_t)(quad * 32) << 16;
        const float scale2 = 0.125f * LOG2E;
        bool ok = true;
        for (int it = 0; ok && it < n; ++it) {
            const int h = g * group + it / per_head, i = j + it % per_head;
            const int tq = i * BLOCK + row;
            const bool live = tq < p.time;
            float delta = 0.f, lse2 = 0.f;
            if (live) {
                const long long at = ((long long)b * p.time + tq) * p.heads + h;
                delta = p.delta[at];
                lse2 = p.lse[at] * LOG2E;
            }
            ok = wait(bar(SP_FULL), (uint32_t)it & 1u);
            if (ok && it > 0) ok = wait(bar(ACC_DONE), (uint32_t)(it - 1) & 1u);
            if (!ok) break;
            tc_fence_after();
            const bool diagonal = i == j;
            {
                const int c = part;
                uint32_t rs[32], rp[32], pp[16], pd[16];
                tmem_ld32(tmem_s + lane_base + c * 32, rs);
                tmem_ld32(tmem_dp + lane_base + c * 32, rp);
                tmem_ld_wait();
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float p0 = 0.f, p1 = 0.f;
                    if (live && !(diagonal && c * 32 + e > row)) p0 = exp2_fast(__uint_as_float(rs[e]) * scale2 - lse2);
                    if (live && !(diagonal && c * 32 + e + 1 > row)) p1 = exp2_fast(__uint_as_float(rs[e + 1]) * scale2 - lse2);
                    pp[e >> 1] = pack2(p0, p1);
                    pd[e >> 1] = pack2(p0 * (__uint_as_float(rp[e]) - delta) * 0.125f, p1 * (__uint_as_float(rp[e + 1]) - delta) * 0.125f);
                }
                store_row32(p_tile, row, c, pp);
                store_row32(ds_tile, row, c, pd);
            }
            fence_async_shared();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(PDS_FULL));
        }
        if (ok) ok = wait(bar(ACC_DONE), (uint32_t)(n - 1) & 1u);
        if (ok) {
            tc_fence_after();
            const int tk = j * BLOCK + row;                     // this thread's key position
            const long long at = ((long long)b * p.time + (tk < p.time ? tk : 0)) * p.kv_heads + g;
            {
                const int which = part >> 1;                                                  // parts 0, 1: dv; parts 2, 3: dk
                uint4* dst = reinterpret_cast<uint4*>((which ? p.out : p.out2) + at * D);
                {
                    const int c = part & 1;
                    uint32_t r[32];
                    tmem_ld32((which ? tmem_dk : tmem_dv) + lane_base + c * 32, r);
                    tmem_ld_wait();
                    if (tk < p.time) {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            dst[c * 4 + e] = make_uint4(pack2(__uint_as_float(r[8 * e]), __uint_as_float(r[8 * e + 1])),
                                                        pack2(__uint_as_float(r[8 * e + 2]), __uint_as_float(r[8 * e + 3])),
                                                        pack2(__uint_as_float(r[8 * e + 4]), __uint_as_float(r[8 * e + 5])),
                                                        pack2(__uint_as_float(r[8 * e + 6]), __uint_as_float(r[8 * e + 7])));
                    }
                }
            }
        }
    }
    linger_after_abort(&s_abort);
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"(512) : "memory");
    }
}

constexpr int FORWARD_SMEM = 5 * TILE_BYTES + 2 * SLAB_BYTES + 128;
constexpr int DQ_KV = 64;
constexpr int DQ_SMEM = 2 * TILE_BYTES + 4 * DQ_KV * 128 + (DQ_KV / 64) * SLAB_BYTES + 128;
constexpr int DKV_SMEM = 1024 + 6 * TILE_BYTES + 4 * SLAB_BYTES + 128;

}  // namespace

int attention_check(const qmoe_attention_t* a, bool backward) {
    if (!a) return fail_arg("attention is null");
    if (a->dim != D) return fail_arg("attention: head width must be 64");
    if (a->dtype != QMOE_BF16) return fail_arg("attention: dtype must be QMOE_BF16");
    if (a->batch <= 0 || a->time <= 0 || a->heads <= 0 || a->kv_heads <= 0 || a->heads % a->kv_heads)
        return fail_arg("attention: sizes must be positive and heads a multiple of kv_heads");
    if ((long long)a->batch * a->time * a->heads * D > (1ll << 40)) return fail_arg("attention: too large");
    if (!a->q || !a->k || !a->v || !a->out || !a->lse) return fail_arg("attention: null buffer address");
    if (backward && (!a->grad_out || !a->delta || !a->dq || !a->dk || !a->dv)) return fail_arg("attention_backward: null buffer address");
    if ((a->q | a->k | a->v | a->out | a->grad_out | a->dq | a->dk | a->dv) & 15u) return fail_arg("attention: buffers must be 16-byte aligned");
    return 0;
}

}  // namespace qmoe

using namespace qmoe;

extern "C" int qmoe_attention_forward(const qmoe_attention_t* a, uint64_t stream_) {
    if (int rc = attention_check(a, false)) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_ATTENTION, stream);
    AttentionParams p = {};
    const uint64_t wide = (uint64_t)a->heads * D, narrow = (uint64_t)a->kv_heads * D;
    if (int rc = make_map_3d(&p.map_q, a->q, wide, (uint64_t)a->time, (uint64_t)a->batch, BLOCK)) return rc;
    if (int rc = make_map_3d(&p.map_k, a->k, narrow, (uint64_t)a->time, (uint64_t)a->batch, BLOCK)) return rc;
    if (int rc = make_map_3d(&p.map_v, a->v, narrow, (uint64_t)a->time, (uint64_t)a->batch, BLOCK)) return rc;
    p.out = (__nv_bfloat16*)a->out; p.lse = (float*)a->lse; p.status = device_status_address();
    p.batch = a->batch; p.time = a->time; p.heads = a->heads; p.kv_heads = a->kv_heads;
    QMOE_CUDA(cudaFuncSetAttribute(attention_forward_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, FORWARD_SMEM));
    const int blocks = (a->time + BLOCK - 1) / BLOCK;
    attention_forward_kernel<<<(unsigned)(blocks * a->heads * a->batch), THREADS, FORWARD_SMEM, stream>>>(p);
    count_tensor_core_launch();
    QMOE_LAUNCH_CHECK("attention_forward_kernel");
    return 0;
}

extern "C" int qmoe_attention_backward(const qmoe_attention_t* a, uint64_t stream_) {
    if (int rc = attention_check(a, true)) return rc;
    cudaStream_t stream = (cudaStream_t)stream_;
    TimedScope timed(KC_ATTENTION, stream);
    AttentionParams p = {};
    const uint64_t wide = (uint64_t)a->heads * D, narrow = (uint64_t)a->kv_heads * D;
    if (int rc = make_map_3d(&p.map_q, a->q, wide, (uint64_t)a->time, (uint64_t)a->batch, BLOCK)) return rc;
    if (int rc = make_map_3d(&p.map_k, a->k, narrow, (uint64_t)a->time, (uint64_t)a->batch, BLOCK)) return rc;
    if (int rc = make_map_3d(&p.map_v, a->v, narrow, (uint64_t)a->time, (uint64_t)a->batch, BLOCK)) return rc;
    if (int rc = make_map_3d(&p.map_do, a->grad_out, wide, (uint64_t)a->time, (uint64_t)a->batch, BLOCK)) return rc;
    p.out_in = (const __nv_bfloat16*)a->out; p.grad_out = (const __nv_bfloat16*)a->grad_out;
    p.lse = (float*)a->lse; p.delta = (float*)a->delta; p.status = device_status_address();
    p.batch = a->batch; p.time = a->time; p.heads = a->heads; p.kv_heads = a->kv_heads;
    const int blocks = (a->time + BLOCK - 1) / BLOCK;
    if (int rc = make_map_3d(&p.map_k2, a->k, narrow, (uint64_t)a->time, (uint64_t)a->batch, DQ_KV)) return rc;
    if (int rc = make_map_3d(&p.map_v2, a->v, narrow, (uint64_t)a->time, (uint64_t)a->batch, DQ_KV)) return rc;
    QMOE_CUDA(cudaFuncSetAttribute(attention_dq_kernel<DQ_KV>, cudaFuncAttributeMaxDynamicSharedMemorySize, DQ_SMEM));
    QMOE_CUDA(cudaFuncSetAttribute(attention_dkv_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DKV_SMEM));
    p.out = (__nv_bfloat16*)a->dq; p.out2 = nullptr;
    attention_dq_kernel<DQ_KV><<<(unsigned)(blocks * a->heads * a->batch), DQ_THREADS, DQ_SMEM, stream>>>(p);
    count_tensor_core_launch();
    QMOE_LAUNCH_CHECK("attention_dq_kernel");
    p.out = (__nv_bfloat16*)a->dk; p.out2 = (__nv_bfloat16*)a->dv;
    attention_dkv_kernel<<<(unsigned)(blocks * a->kv_heads * a->batch), DKV_THREADS, DKV_SMEM, stream>>>(p);
    count_tensor_core_launch();
    QMOE_LAUNCH_CHECK("attention_dkv_kernel");
    return 0;
}
