// Grouped expert GEMMs on the 5th-generation tensor cores (sm_100a): tcgen05.mma with bf16
// operands staged in shared memory by TMA (cp.async.bulk.tensor, 128-byte swizzle, no multicast),
// fp32 accumulators in tensor memory (TMEM), read back with tcgen05.ld for the epilogue.
//
// One persistent kernel, one CTA per SM, 10 warps; the expert products run as CTA PAIRS (CTAS = 2: the two
// CTAs of a cluster share one 256 x 256 tile, tcgen05.mma.cta_group::2), the small router products with one
// CTA per 128 x 256 tile:
//   warp 0      TMA producer (one lane): fills a ring of {A 128x64, B 256x64 or this CTA's 128x64 half} bf16
//               tiles (4 stages of 48 KiB, or 6 stages of 32 KiB per CTA of a pair; two fewer in dSwiGLU, whose
//               epilogue stages its own operands in shared memory)
//   warp 1      MMA issuer (one lane, in a pair only the first CTA's): 4 x tcgen05.mma (K = 16 each) per
//               stage, commits free the stage in both CTAs; also allocates / frees the 512 TMEM columns
//               (two 128x256 fp32 accumulators per CTA)
//   warps 2-9   epilogue: two warps per 32-lane TMEM quadrant (= 32 tile rows), each taking half of
//               the columns; they convert and store to HBM while the MMA warp already works on the
//               next tile in the other accumulator
//
// Three problem kinds share the kernel (template MODE):
//   MODE_PLAIN   C[rows, N] (bf16) = A[rows, K] . B_e  (+ A2 . B2_e), rows in the dispatched layout,
//                the expert e of a 128-row tile picks the weight slab.  B either [E*N, K] (K-major,
//                "x W^T") or [E*K, N] (MN-major, "g W").
//   MODE_SWIGLU  G = X Wg_e^T, U = X Wu_e^T (128 + 128 accumulator columns), H = silu(G) * U, all
//                three stored as bf16.
//   MODE_DSWIGLU dH = dY Wd_e (never stored): dU = dH * silu(G), dG = dH * U * silu'(G), bf16; G and U are
//                fetched and dG and dU written by TMA in the layout the accumulator is read in.
//   MODE_WGRAD   C_e[M, N] (fp32) = A_e^T . B_e, contraction over the rows of expert e (both
//                operands MN-major); experts without rows are skipped and their slab is not written.
//                Up to three such products of one shape share a launch (dWd, dWg, dWu).
//   MODE_ROUTER / MODE_PLAIN_F32: the router's products (fp32 results from bf16 terms), one row group.
//
// Every wait on an mbarrier is bounded (about one second of %globaltimer); when one runs out the
// CTA records a code in the status word, stops issuing work, waits a bounded time for copies in
// flight, meets its partner CTA at the cluster barrier (pairs), frees its TMEM and returns.
#include <cuda.h>

#include <map>
#include <mutex>
#include <tuple>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace qmoe {

namespace {

constexpr int BM = 128, BN = 256, BK = 64, UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;   // 16 KiB: the 128 rows (or 128 MN columns) this CTA contributes
constexpr int CHUNK_BYTES = 64 * BK * 2;     // one 64 x 64 bf16 TMA box (8 KiB)
// CTAS = 1: one CTA owns a 128 x 256 tile (A 16 KiB + B 32 KiB per stage, 4 stages).
// CTAS = 2: a pair of CTAs (cluster of 2, tcgen05 cta_group::2) owns a 256 x 256 tile; each CTA stages its 128
//           rows of A and HALF of B (16 + 16 KiB per stage, 6 stages), so every byte fetched from L2 feeds
//           1.5x more math, and the issuing CTA's MMA reads both halves.
// Shared memory of a CTA: [operand ring][epilogue staging, one slice per epilogue warp][mbarriers].  The dSwiGLU
// epilogue keeps two {G, U} pairs of 32-row x 64-column boxes for every two warps that share rows (fetched and written
// back by TMA), which costs the ring a stage; the other modes only need a small transpose buffer per warp.
constexpr int EPILOGUE_WARPS = 8;
constexpr int NUM_THREADS = 64 + 32 * EPILOGUE_WARPS + 32;  // TMA warp for A, MMA warp, epilogue warps, TMA warp for B
constexpr int B_PRODUCER_WARP = 2 + EPILOGUE_WARPS;
constexpr int MODE_DSWIGLU_ID = 3;
constexpr int BOX_BYTES = 32 * 64 * 2;            // one 32 x 64 bf16 box of the dSwiGLU epilogue (4 KiB, 128-byte rows)
constexpr int BARRIER_BYTES = 512;
template <int CTAS, int MODE> struct Cfg {
    static constexpr bool STAGED = MODE == MODE_DSWIGLU_ID;
    static constexpr int STAGES = CTAS == 2 ? (STAGED ? 5 : 6) : (STAGED ? 3 : 4);
    static constexpr int B_STAGE_BYTES = (CTAS == 2 ? BN / 2 : BN) * BK * 2;
    static constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
    static constexpr int EPI_WARP_BYTES = 32 * 80;            // transpose buffer of one epilogue warp (not dSwiGLU)
    static constexpr int EPI_SLICE_BYTES = 4 * BOX_BYTES;     // dSwiGLU: two {G, U} buffers for each two warps on the same rows
    static constexpr int EPI_BYTES = STAGED ? (EPILOGUE_WARPS / 2) * EPI_SLICE_BYTES : EPILOGUE_WARPS * EPI_WARP_BYTES;  // a multiple of 1 KiB either way
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /*alignment slack*/ + EPI_BYTES + BARRIER_BYTES;
};
constexpr uint32_t TMEM_COLS = 512;

enum { MODE_PLAIN = 0, MODE_SWIGLU = 1, MODE_WGRAD = 2, MODE_DSWIGLU = MODE_DSWIGLU_ID, MODE_ROUTER = 4, MODE_PLAIN_F32 = 5 };
enum { STATUS_WAIT_PRODUCER = 101, STATUS_WAIT_MMA = 102, STATUS_WAIT_EPILOGUE = 103 };

struct alignas(64) GemmParams {
    CUtensorMap map_a, map_b, map_a2, map_b2;
    CUtensorMap map_a3, map_b3;  // WGRAD with three problems in one launch: operands of problems 0, 1, 2 = (a, b), (a2, b2), (a3, b3)
    const int* offsets;   // [E + 1] first dispatched row of each expert
    const int* counts;    // [E]
    int* status;
    void* out0;           // PLAIN: C bf16; SWIGLU: G; WGRAD: C fp32 (stacked per expert); DSWIGLU: dG
    void* out1;           // SWIGLU: U; DSWIGLU: dU
    void* out2;           // SWIGLU: H
    const void* in0;      // DSWIGLU: G (saved by the forward)
    const void* in1;      // DSWIGLU: U
    long long ldc;        // row pitch of the outputs, in elements
    long long c_slab;     // WGRAD: elements per expert
    int experts;
    int n_tiles;          // PLAIN/WGRAD: ceil(N / 256); SWIGLU: ceil(N / 128)
    int m_tiles;          // WGRAD: ceil(M / 128)
    int M, N, K;          // WGRAD: M, N of one expert's output; others: N = output columns, K = inner size of one segment
    int b_rows;           // rows of the stacked B operand per expert
    int segments;         // 1, or 2 when (A2, B2) is accumulated into the same tile
    // PLAIN with scatter: row r of the output is not stored at out0 + r * ldc but sent to the rank and row
    // recorded for it (return address = rank << 26 | row), i.e. straight into that GPU's buffer
    const int* scatter_ret;              // [rows] return addresses, or null for a plain store
    unsigned long long scatter_base[16]; // every rank's destination buffer (own entry: local address)
    int scatter_wide;     // scatter in 256-byte row pieces (0: 64-byte pieces)
    int plain_rows;       // > 0: one group of this many rows instead of the expert groups of `offsets`
    int transpose_out;    // WGRAD: bit i set = problem i stores the [M, N] product of each expert as [N, M]
    int problems;         // WGRAD: 1, or 3 products of the same shape (outputs out0, out1, out2) sharing the tile queue
    int group_stride;     // ROUTER: accumulator columns [0,S), [S,2S), [2S,3S) hold the three bf16 terms of the weights
};

struct Tile {
    int expert, row0, n0, kblocks, krow0;
    int problem;      // WGRAD: which of the launch's products this tile belongs to
    int bn;           // accumulator columns of this tile: 256, or 128 for a last tile that is at most half full (B in MN-major only)
    bool valid;       // false: nothing to do for the whole tile (all CTAs of the tile skip it)
    bool rows_valid;  // CTAS == 2: false when this CTA's 128 rows lie past the end of the expert (compute, do not store)
};

// First 128-row tile of each expert: a table in shared memory, except where the epilogue's boxes leave no room for it
// (dSwiGLU on CTA pairs) and the two values a tile needs come from the offsets in global memory instead.
template <bool IN_SHARED> struct StartTable {
    const int* shared;
    const int* offsets;
    __device__ __forceinline__ int operator[](int e) const { return IN_SHARED ? shared[e] : __ldg(offsets + e) / kRowPad; }
};
template <int MODE, int CTAS> constexpr bool starts_in_shared() { return !(MODE == MODE_DSWIGLU && CTAS == 2); }

// s_start[e]: first 128-row tile of expert e.  s_pair[e] (CTAS == 2): first 256-row pair-tile of expert e, an
// expert with an odd number of 128-row tiles gets a last pair-tile whose second half is not stored.
template <int MODE, bool B_MN, int CTAS>
__device__ __forceinline__ Tile decode_tile(const GemmParams& p, const StartTable<starts_in_shared<MODE, CTAS>()>& s_start,
                                            const int* s_pair, const int* s_order, int t, int cta_rank) {
    Tile tile;
    tile.valid = true;
    tile.rows_valid = true;
    tile.problem = 0;
    if (MODE == MODE_WGRAD) {
        // m_tiles counts CTAS * 128-row groups of the output.  Inside an expert the tiles run product by product
        // (dWg, dWu, dWd: the first two share the layer input), every tile of a product side by side: the grid then
        // streams each operand panel from HBM once while its tiles walk the contraction in step.  (Dealing the
        // products out tile by tile instead makes every wave of the grid touch all panels of the row-side operands
        // and read them again in the next wave: measured 2.5 to 9 % slower at 64 experts, the same at 8.)
        const int per_product = p.m_tiles * p.n_tiles, per = per_product * p.problems;
        const int slot = t / per;
        int rem = t - slot * per;
        const int turn = rem / per_product;                      // 0, 1, 2 -> problems 1, 2, 0
        tile.problem = p.problems == 3 ? (turn + 1) % 3 : turn;
        rem -= turn * per_product;
        const int e = s_order[slot];
        tile.expert = e;
        tile.row0 = (rem % p.m_tiles) * (BM * CTAS) + cta_rank * BM;
        tile.n0 = (rem / p.m_tiles) * BN;
        const int count = p.counts[e];
        tile.kblocks = (count + BK - 1) / BK;
        tile.krow0 = s_start[e] * kRowPad;
        tile.valid = count > 0;
    } else {
        // tiles are numbered from the first group's first row (a caller may pass a sub-range of the
        // experts, whose offsets do not start at row 0)
        auto first_of = [&](int e) { return CTAS == 2 ? s_pair[e] : s_start[e]; };
        const int first = first_of(0);
        int lo = 0, hi = p.experts;  // largest e with (first_of(e) - first) * n_tiles <= t
        while (hi - lo > 1) {
            const int mid = (lo + hi) >> 1;
            if ((long long)(first_of(mid) - first) * p.n_tiles <= t) lo = mid; else hi = mid;
        }
        const int e = lo;
        const int groups = first_of(e + 1) - first_of(e);
        const int local = t - (first_of(e) - first) * p.n_tiles;
        const int m_tile = (local % groups) * CTAS + cta_rank;  // 128-row tile inside the expert
        const int start = s_start[e];
        tile.expert = e;
        tile.row0 = (start + m_tile) * BM;
        tile.rows_valid = m_tile < s_start[e + 1] - start;
        tile.n0 = (local / groups) * (MODE == MODE_SWIGLU ? 128 : BN);
        tile.kblocks = ((p.K + BK - 1) / BK) * p.segments;
        tile.krow0 = 0;
    }
    // MN-major B arrives in 64-column boxes, so a narrow last tile simply loads and multiplies half of them
    tile.bn = (B_MN && MODE != MODE_SWIGLU && p.N - tile.n0 <= BN / 2) ? BN / 2 : BN;
    return tile;
}

// 1 / (1 + 2^(-v log2 e)) with the approximate exp2 / reciprocal units (relative error ~1e-6,
// far below one bf16 ulp); saturates cleanly to 0 and 1 for large |v|
__device__ __forceinline__ float fast_sigmoid(float v) {
    float e, r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(e) : "f"(-1.4426950408889634f * v));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(1.0f + e));
    return r;
}
__device__ __forceinline__ float bf16_lo(uint32_t w) { return __uint_as_float(w << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t w) { return __uint_as_float(w & 0xffff0000u); }

__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t*>(&h);
}

// store 32 consecutive bf16 of one row; `valid` = number of columns inside the matrix
__device__ __forceinline__ void store_row32_bf16(__nv_bfloat16* dst, const float* v, int valid) {
    if (valid >= 32) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            uint4 w = make_uint4(pack_bf16(v[8 * q], v[8 * q + 1]), pack_bf16(v[8 * q + 2], v[8 * q + 3]),
                                 pack_bf16(v[8 * q + 4], v[8 * q + 5]), pack_bf16(v[8 * q + 6], v[8 * q + 7]));
            *reinterpret_cast<uint4*>(dst + 8 * q) = w;
        }
    } else {
#pragma unroll
        for (int i = 0; i < 32; ++i)
            if (i < valid) dst[i] = __float2bfloat16_rn(v[i]);
    }
}

// Per-warp transpose buffer: 32 rows of 64 bytes, row pitch 80 bytes (keeps 16-byte alignment and
// spreads the rows over the banks).
constexpr int STAGE_PITCH = 80;
constexpr int EPI_STAGE_BYTES = 32 * STAGE_PITCH;

// Thread `lane` holds 32 consecutive bf16 (16 packed words) of row `lane`.  Write the 32 x 32 block to
// global memory (dst = first element of the block, row pitch ldc elements) so that every store
// instruction covers 8 rows x 64 contiguous bytes.
__device__ __forceinline__ void store_block32(uint32_t stage, int lane, const uint32_t* w, __nv_bfloat16* dst, long long ldc) {
    const uint32_t mine = stage + lane * STAGE_PITCH;
#pragma unroll
    for (int q = 0; q < 4; ++q)
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(mine + 16 * q), "r"(w[4 * q]), "r"(w[4 * q + 1]),
                     "r"(w[4 * q + 2]), "r"(w[4 * q + 3]) : "memory");
    __syncwarp();
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int row = j * 8 + (lane >> 2), piece = lane & 3;
        uint4 v;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "r"(stage + row * STAGE_PITCH + 16 * piece) : "memory");
        *reinterpret_cast<uint4*>(dst + (long long)row * ldc + piece * 8) = v;
    }
    __syncwarp();
}

// Same transpose, but every row has its own destination: `dst_row` is THIS lane's row pointer (null =
// skip the row, e.g. a pad row); the pointer of the row a lane stores is fetched by shuffle.
__device__ __forceinline__ void scatter_block32(uint32_t stage, int lane, const uint32_t* w, __nv_bfloat16* dst_row) {
    const uint32_t mine = stage + lane * STAGE_PITCH;
#pragma unroll
    for (int q = 0; q < 4; ++q)
        asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(mine + 16 * q), "r"(w[4 * q]), "r"(w[4 * q + 1]),
                     "r"(w[4 * q + 2]), "r"(w[4 * q + 3]) : "memory");
    __syncwarp();
    const unsigned long long mine_ptr = (unsigned long long)dst_row;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int row = j * 8 + (lane >> 2), piece = lane & 3;
        const unsigned long long base = __shfl_sync(0xffffffffu, mine_ptr, row);
        uint4 v;
        asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                     : "r"(stage + row * STAGE_PITCH + 16 * piece) : "memory");
        if (base) *reinterpret_cast<uint4*>((__nv_bfloat16*)base + piece * 8) = v;
    }
    __syncwarp();
}

// Thread `lane` holds the 32 fp32 values of row `lane`; store the 32 x 32 block to `dst` (first element of the
// block, row pitch ldc floats, rows >= rows_left skipped) so that every store instruction covers 8 rows x 64
// contiguous bytes.  Two passes of 16 columns through the 32 x 80 B staging buffer.
__device__ __forceinline__ void store_block32_f32(uint32_t stage, int lane, const uint32_t* r, float* dst, long long ldc,
                                                  long long rows_left) {
    const uint32_t mine = stage + lane * STAGE_PITCH;
#pragma unroll
    for (int s = 0; s < 2; ++s) {
#pragma unroll
        for (int q = 0; q < 4; ++q)
            asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(mine + 16 * q), "r"(r[16 * s + 4 * q]),
                         "r"(r[16 * s + 4 * q + 1]), "r"(r[16 * s + 4 * q + 2]), "r"(r[16 * s + 4 * q + 3]) : "memory");
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int row = j * 8 + (lane >> 2), piece = lane & 3;
            uint4 v;
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                         : "r"(stage + row * STAGE_PITCH + 16 * piece) : "memory");
            if (row < rows_left) *reinterpret_cast<uint4*>(dst + (long long)row * ldc + 16 * s + 4 * piece) = v;
        }
        __syncwarp();
    }
}

// Scatter of 128 columns: thread `lane` holds 128 consecutive bf16 (64 packed words) of row `lane`, every row
// has its own destination (`dst_row`, null = skip).  Rows that live on another GPU cross NVLink, where a
// store of 64 contiguous bytes per row costs about twice the time per byte of a long one, so the block goes
// through the staging buffer 8 rows at a time and every store instruction covers 2 rows x 256 contiguous bytes.
__device__ __forceinline__ void scatter_rows256(uint32_t stage, int lane, const uint32_t* w, __nv_bfloat16* dst_row) {
    constexpr int PITCH = 272;  // 8 rows x 272 B fit the 32 x 80 B buffer; 68 words per row keep the v4 accesses conflict-free
    const unsigned long long mine_ptr = (unsigned long long)dst_row;
#pragma unroll
    for (int pass = 0; pass < 4; ++pass) {
        if ((lane >> 3) == pass) {
            const uint32_t mine = stage + (lane & 7) * PITCH;
#pragma unroll
            for (int q = 0; q < 16; ++q)
                asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(mine + 16 * q), "r"(w[4 * q]), "r"(w[4 * q + 1]),
                             "r"(w[4 * q + 2]), "r"(w[4 * q + 3]) : "memory");
        }
        __syncwarp();
#pragma unroll
        for (int it = 0; it < 4; ++it) {
            const int row = it * 2 + (lane >> 4), piece = lane & 15;
            const unsigned long long base = __shfl_sync(0xffffffffu, mine_ptr, pass * 8 + row);
            uint4 v;
            asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                         : "r"(stage + row * PITCH + 16 * piece) : "memory");
            if (base) *reinterpret_cast<uint4*>((__nv_bfloat16*)base + piece * 8) = v;
        }
        __syncwarp();
    }
}

// CTAS == 2: two CTAs of a cluster (a CTA pair on neighbouring SMs) share one 256-row x 256-column tile.
// Each stages its own 128 rows of A and half of the B tile, the pair's first CTA issues one
// cta_group::2 MMA per k-step that reads both halves, and each CTA converts the 128 x 256 accumulator
// that lands in its own tensor memory.  Per SM and k-step that is 32 KiB of operands instead of 48 KiB.
template <int MODE, bool A_MN, bool B_MN, int CTAS>
__global__ void __launch_bounds__(NUM_THREADS, 1)
grouped_gemm_kernel(const __grid_constant__ GemmParams p) {
    using Config = Cfg<CTAS, MODE>;
    constexpr int STAGES = Config::STAGES, B_STAGE_BYTES = Config::B_STAGE_BYTES, STAGE_BYTES = Config::STAGE_BYTES;
    extern __shared__ uint8_t smem_raw[];
    constexpr bool STARTS_IN_SHARED = starts_in_shared<MODE, CTAS>();
    __shared__ int s_start_table[STARTS_IN_SHARED ? kMaxExperts + 1 : 1];  // first 128-row tile of each expert
    const StartTable<STARTS_IN_SHARED> s_start{s_start_table, p.offsets};
    __shared__ int s_pair[kMaxExperts + 1];   // CTAS == 2: first 256-row pair-tile of each expert
    __shared__ int s_order[kMaxExperts];      // WGRAD: experts by decreasing row count (ties by index)
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cta_rank = CTAS == 2 ? (int)cluster_ctarank() : 0;
    const int first_tile = CTAS == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;  // a cluster is two consecutive blocks
    const int tile_stride = (int)gridDim.x / CTAS;
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t epi0 = base + STAGES * STAGE_BYTES;   // epilogue staging, 1 KiB aligned
    const uint32_t bars = epi0 + Config::EPI_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto tfull_bar = [&](int a) { return bars + 8u * (2 * STAGES + a); };
    auto tempty_bar = [&](int a) { return bars + 8u * (2 * STAGES + 2 + a); };

    if (!STARTS_IN_SHARED) {
        // nothing to fill: the table reads the offsets
    } else if (p.plain_rows > 0) {
        if (threadIdx.x == 0) { s_start_table[0] = 0; s_start_table[1] = (p.plain_rows + kRowPad - 1) / kRowPad; }
    } else {
        for (int i = threadIdx.x; i <= p.experts; i += NUM_THREADS) s_start_table[i] = p.offsets[i] / kRowPad;
    }
    if (MODE == MODE_WGRAD) {
        // Tiles of large experts cost more (longer contraction).  Walking the experts from large to
        // small and dealing tiles round-robin gives every CTA the same mix of long and short tiles.
        for (int i = threadIdx.x; i < p.experts; i += NUM_THREADS) {
            const int mine = p.counts[i];
            int rank = 0;
            for (int j = 0; j < p.experts; ++j) {
                const int other = p.counts[j];
                rank += (other > mine || (other == mine && j < i)) ? 1 : 0;
            }
            s_order[rank] = i;
        }
    }
    if (threadIdx.x == 0) {
        s_abort = 0;
        // CTAS == 2: the copies of both CTAs count on the first CTA's full barrier; the MMA issuer (first
        // CTA) releases a stage and publishes an accumulator on the barriers of both; the epilogue warps
        // of both hand an accumulator back on the first CTA's barrier
        for (int s = 0; s < STAGES; ++s) { mbar_init(full_bar(s), 1); mbar_init(empty_bar(s), 1); }
        for (int a = 0; a < 2; ++a) { mbar_init(tfull_bar(a), 1); mbar_init(tempty_bar(a), EPILOGUE_WARPS * CTAS); }
        if (MODE == MODE_DSWIGLU) {  // per two warps on the same rows: for each buffer "loaded" and "second half written"
            for (int i = 0; i < 2 * EPILOGUE_WARPS; ++i) mbar_init(bars + 8u * (2 * STAGES + 4 + i), 1);
            prefetch_map(&p.map_a2); prefetch_map(&p.map_b2); prefetch_map(&p.map_a3); prefetch_map(&p.map_b3);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        prefetch_map(&p.map_a);
        prefetch_map(&p.map_b);
        if (MODE == MODE_SWIGLU || (MODE != MODE_DSWIGLU && p.segments == 2)) prefetch_map(&p.map_b2);
        if (MODE != MODE_DSWIGLU && p.segments == 2) prefetch_map(&p.map_a2);
    }
    if (warp == 1) {
        if (CTAS == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(&s_tmem_base)), "r"(TMEM_COLS) : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (CTAS == 2) {
        // pair-tiles of the experts before e; an odd last 128-row tile takes a pair-tile of its own
        for (int i = threadIdx.x; i <= p.experts; i += NUM_THREADS) {
            int sum = 0;
            for (int j = 0; j < i; ++j) sum += (s_start[j + 1] - s_start[j] + 1) >> 1;
            s_pair[i] = sum;
        }
        __syncthreads();
        cluster_sync();  // the partner's barriers exist before anything arrives on them
    }
    tc_fence_after();
    const uint32_t tmem_base = s_tmem_base;

    int total_tiles;
    if (MODE == MODE_WGRAD) total_tiles = p.experts * p.m_tiles * p.n_tiles * p.problems;
    else if (CTAS == 2) total_tiles = s_pair[p.experts] * p.n_tiles;
    else total_tiles = (s_start[p.experts] - s_start[0]) * p.n_tiles;
    volatile int* abort_flag = &s_abort;

    if (warp == 0 || warp == B_PRODUCER_WARP) {
        // ------------------------------ TMA producers -----------------------------
        // Two threads: one asks for the A boxes of every stage (and announces the stage's bytes), the other for the B
        // boxes.  Issuing a TMA instruction costs its thread of the order of a hundred cycles whatever the box holds;
        // with announce + A + B in one thread a k-block took that thread longer than its 512 cycles of tensor work.
        const bool does_a = warp == 0;
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            for (int t = first_tile; t < total_tiles && !*abort_flag; t += tile_stride) {
                const Tile tile = decode_tile<MODE, B_MN, CTAS>(p, s_start, s_pair, s_order, t, cta_rank);
                if (!tile.valid) continue;
                const int kb_per_seg = tile.kblocks / (MODE == MODE_WGRAD ? 1 : p.segments);
                for (int kb = 0; kb < tile.kblocks; ++kb) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, STATUS_WAIT_PRODUCER); }
                        break;
                    }
                    const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_STAGE_BYTES;
                    // CTAS == 2: both CTAs' bytes are expected (and counted) on the first CTA's barrier
                    const uint32_t bar = CTAS == 2 ? map_to_cta(full_bar(stage), 0) : full_bar(stage);
                    const int bn_mine = tile.bn / CTAS;      // columns of the B tile this CTA stages
                    const uint32_t stage_bytes = A_STAGE_BYTES + (uint32_t)bn_mine * BK * 2;
                    if (does_a) {
                        if (CTAS == 1) mbar_expect_tx(bar, stage_bytes);
                        else if (cta_rank == 0) mbar_expect_tx(full_bar(stage), 2 * stage_bytes);
                    }
                    auto load = [&](const CUtensorMap* map, uint32_t dst, int c0, int c1) {
                        if (CTAS == 2) tma_load_2d_pair(map, dst, bar, c0, c1);
                        else tma_load_2d(map, dst, bar, c0, c1);
                    };
                    const int n_mine = tile.n0 + cta_rank * bn_mine;
                    if (MODE == MODE_WGRAD) {
                        const int krow = tile.krow0 + kb * BK;
                        const CUtensorMap* ma = tile.problem == 0 ? &p.map_a : tile.problem == 1 ? &p.map_a2 : &p.map_a3;
                        const CUtensorMap* mb = tile.problem == 0 ? &p.map_b : tile.problem == 1 ? &p.map_b2 : &p.map_b3;
                        if (does_a) {
#pragma unroll
                            for (int j = 0; j < BM / 64; ++j) load(ma, sa + j * CHUNK_BYTES, tile.row0 + 64 * j, krow);
                        } else {
#pragma unroll
                            for (int j = 0; j < BN / CTAS / 64; ++j)
                                if (64 * j < bn_mine) load(mb, sb + j * CHUNK_BYTES, n_mine + 64 * j, krow);
                        }
                    } else {
                        const int seg = kb / kb_per_seg;
                        const int k0 = (kb - seg * kb_per_seg) * BK;
                        const CUtensorMap* ma = seg ? &p.map_a2 : &p.map_a;
                        const CUtensorMap* mb = seg ? &p.map_b2 : &p.map_b;
                        // A is K-major in these modes.  The unused half of an odd pair-tile reads past the end of
                        // the matrix: TMA fills zeros without touching memory, and a tensor core fed zeros draws
                        // far less power than one fed another expert's rows (the result is discarded either way).
                        if (does_a) {
                            load(ma, sa, k0, (CTAS == 2 && !tile.rows_valid) ? 0x3fffff00 : tile.row0);
                        } else if (MODE == MODE_SWIGLU) {
                            // accumulator columns [0, 128) = gate, [128, 256) = up; a pair splits them between its CTAs
                            if (CTAS == 2) {
                                load(cta_rank ? &p.map_b2 : &p.map_b, sb, k0, tile.expert * p.b_rows + tile.n0);
                            } else {
                                load(&p.map_b, sb, k0, tile.expert * p.b_rows + tile.n0);
                                load(&p.map_b2, sb + B_STAGE_BYTES / 2, k0, tile.expert * p.b_rows + tile.n0);
                            }
                        } else if (B_MN) {
#pragma unroll
                            for (int j = 0; j < BN / CTAS / 64; ++j)
                                if (64 * j < bn_mine) load(mb, sb + j * CHUNK_BYTES, n_mine + 64 * j, tile.expert * p.b_rows + k0);
                        } else {
                            load(mb, sb, k0, tile.expert * p.b_rows + n_mine);
                        }
                    }
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        if (lane == 0 && cta_rank == 0) {
            int stage = 0;
            uint32_t phase = 0;
            int iter = 0;
            // a pair's commit reaches the barrier of both CTAs
            auto commit = [&](uint32_t bar) {
                if (CTAS == 2) umma_commit_both(bar);
                else umma_commit(bar);
            };
            for (int t = first_tile; t < total_tiles && !*abort_flag; t += tile_stride) {
                const Tile tile = decode_tile<MODE, B_MN, CTAS>(p, s_start, s_pair, s_order, t, cta_rank);
                if (!tile.valid) continue;
                const int acc = iter & 1;
                const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
                bool ok = mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag);
                tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)acc * BN;
                const uint32_t idesc = make_idesc<A_MN, B_MN, BM * CTAS>(tile.bn);
                bool ready = false;   // the stage of this k-block was seen full while the k-block before it was issued
                for (int kb = 0; ok && kb < tile.kblocks; ++kb) {
                    if (!ready) {
                        ok = mbar_wait(full_bar(stage), phase, abort_flag);
                        if (!ok) break;
                    }
                    tc_fence_after();
                    const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_STAGE_BYTES;
                    int next_stage = stage + 1;
                    uint32_t next_phase = phase;
                    if (next_stage == STAGES) { next_stage = 0; next_phase ^= 1u; }
#pragma unroll
                    for (int kk = 0; kk < BK / UMMA_K; ++kk) {
                        // K-major: 128-byte rows, 8-row groups 1024 B apart, +32 B per 16 k.
                        // MN-major: 64-wide chunks 8 KiB apart (LBO), 8-k groups 1024 B apart, +2 KiB per 16 k.
                        const uint64_t adesc = A_MN ? make_desc(sa + kk * 2048, CHUNK_BYTES, 1024)
                                                    : make_desc(sa + kk * 32, 16, 1024);
                        const uint64_t bdesc = B_MN ? make_desc(sb + kk * 2048, CHUNK_BYTES, 1024)
                                                    : make_desc(sb + kk * 32, 16, 1024);
                        // the look at the next stage's barrier goes between the MMAs, where the tensor pipe has work queued,
                        // rather than after the last one, where its latency would leave the pipe idle
                        if (kk == BK / UMMA_K - 1) ready = kb + 1 < tile.kblocks && mbar_try(full_bar(next_stage), next_phase);
                        if (CTAS == 2) umma_bf16_pair(tmem_d, adesc, bdesc, idesc, (kb | kk) ? 1u : 0u);
                        else umma_bf16(tmem_d, adesc, bdesc, idesc, (kb | kk) ? 1u : 0u);
                    }
                    commit(empty_bar(stage));  // the stage is free once these MMAs have read it
                    stage = next_stage; phase = next_phase;
                }
                if (!ok) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, STATUS_WAIT_MMA); }
                    break;
                }
                commit(tfull_bar(acc));
                ++iter;
            }
        }
    } else if (MODE == MODE_DSWIGLU) {
        // ------------------------------ epilogue of dSwiGLU -------------------------
        // dG = dH . U . silu'(G), dU = dH . silu(G), with dH only ever in tensor memory.  G and U arrive, and dG and
        // dU leave, through TMA in boxes of 32 rows x 64 columns laid out like the accumulator is read (one thread =
        // one row; 128-byte rows under the 128-byte swizzle, so the rows of a quarter warp fall on different banks):
        // no transposes and no per-thread global accesses.  Full 128-byte rows matter: the same bytes moved as 64-byte
        // rows took twice the TMA requests and slowed the operand feed of the main loop by a tenth.  The two warps
        // that read the same 32 lanes of tensor memory share two {G, U} buffers and split every box between them,
        // columns 0-31 and 32-63: the first of the two (the leader) asks for the boxes and stores them, the second
        // tells it through a barrier when its half is written.  While a chunk is worked on, the boxes of the next
        // (of this tile or of the pair's next tile) are already on their way, and results overwrite their inputs in
        // place before the store.
        const int warp_e = warp - 2, quad = warp & 3, slot = warp_e & 3, side = warp_e >> 2;
        const bool leader = side == 0;
        const uint32_t slice = epi0 + (uint32_t)slot * Config::EPI_SLICE_BYTES;
        auto load_bar = [&](uint32_t n) { return bars + 8u * (2 * STAGES + 4 + slot * 4 + (n & 1u)); };
        auto half_done_bar = [&](uint32_t n) { return bars + 8u * (2 * STAGES + 4 + slot * 4 + 2 + (n & 1u)); };
        auto buffer = [&](uint32_t n) { return slice + (n & 1u) * 2u * BOX_BYTES; };
        // chunks [0, c_last) of 64 columns these warps convert in `tile` (none when their rows lie past the expert's end)
        auto chunks_of = [&](const Tile& tile) {
            if (!tile.valid || (CTAS == 2 && !tile.rows_valid)) return 0;
            const int in_tile = tile.bn / 64, in_range = (p.N - tile.n0 + 63) / 64;
            return in_tile < in_range ? in_tile : in_range;
        };
        auto issue_load = [&](const Tile& tile, int c, uint32_t n) {  // one lane: boxes of chunk c into buffer n & 1
            const uint32_t bar = load_bar(n), dst = buffer(n);
            const int col = tile.n0 + c * 64, row = tile.row0 + quad * 32;
            mbar_expect_tx(bar, 2 * BOX_BYTES);
            tma_load_2d(&p.map_a2, dst, bar, col, row);
            tma_load_2d(&p.map_b2, dst + BOX_BYTES, bar, col, row);
        };
        uint32_t n = 0;            // chunks consumed: buffer n & 1, barrier phase (n >> 1) & 1
        bool on_its_way = false;   // leader: the boxes of chunk number n have been asked for
        int iter = 0;
        bool gave_up = false;
        for (int t = first_tile; t < total_tiles && !*abort_flag && !gave_up; t += tile_stride) {
            const Tile tile = decode_tile<MODE, B_MN, CTAS>(p, s_start, s_pair, s_order, t, cta_rank);
            if (!tile.valid) continue;
            const int c_end = chunks_of(tile);
            if (leader && c_end > 0 && !on_its_way) {  // only the first chunk of the kernel is not prefetched
                if (lane == 0) issue_load(tile, 0, n);
                on_its_way = true;
            }
            const int acc = iter & 1;
            const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) {
                if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, STATUS_WAIT_EPILOGUE); }
                break;
            }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)acc * BN + (uint32_t)side * 32u;
#pragma unroll 1
            for (int c = 0; c < c_end; ++c) {
                uint32_t r[32];
                tmem_ld32(taddr + c * 64, r);
                if (leader) {
                    // the chunk after this one: the next of this tile, else the first of the next tile with work
                    Tile next_tile = tile;
                    int next_c = c + 1, next_last = c_end;
                    if (next_c >= c_end) {
                        next_c = next_last = 0;
                        for (int u = t + tile_stride; u < total_tiles; u += tile_stride) {
                            next_tile = decode_tile<MODE, B_MN, CTAS>(p, s_start, s_pair, s_order, u, cta_rank);
                            next_last = chunks_of(next_tile);
                            if (next_last > 0) break;
                        }
                    }
                    on_its_way = next_c < next_last;
                    if (on_its_way && lane == 0) {
                        bulk_wait_read_all();   // the store that last used that buffer (chunk n - 1) has read it
                        issue_load(next_tile, next_c, n + 1);
                    }
                }
                tmem_ld_wait();
                if (!mbar_wait(load_bar(n), (n >> 1) & 1u, abort_flag)) {
                    if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, STATUS_WAIT_EPILOGUE); }
                    gave_up = true;
                    break;
                }
                const uint32_t row_g = buffer(n) + (uint32_t)lane * 128u, row_u = row_g + BOX_BYTES;
                const uint32_t twist = (uint32_t)lane & 7u;   // 128-byte swizzle: 16-byte piece j of row r sits at j ^ (r & 7)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const uint32_t at = ((uint32_t)(4 * side + j) ^ twist) * 16u;
                    uint32_t gw[4], uw[4], og[4], ou[4];
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(gw[0]), "=r"(gw[1]), "=r"(gw[2]), "=r"(gw[3]) : "r"(row_g + at) : "memory");
                    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(uw[0]), "=r"(uw[1]), "=r"(uw[2]), "=r"(uw[3]) : "r"(row_u + at) : "memory");
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float g0 = bf16_lo(gw[i]), g1 = bf16_hi(gw[i]);
                        const float u0 = bf16_lo(uw[i]), u1 = bf16_hi(uw[i]);
                        const float s0 = fast_sigmoid(g0), s1 = fast_sigmoid(g1);
                        const float h0 = __uint_as_float(r[8 * j + 2 * i]), h1 = __uint_as_float(r[8 * j + 2 * i + 1]);
                        ou[i] = pack_bf16(h0 * g0 * s0, h1 * g1 * s1);
                        og[i] = pack_bf16(h0 * u0 * s0 * (1.f + g0 * (1.f - s0)), h1 * u1 * s1 * (1.f + g1 * (1.f - s1)));
                    }
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(row_g + at), "r"(og[0]), "r"(og[1]), "r"(og[2]), "r"(og[3]) : "memory");
                    asm volatile("st.shared.v4.u32 [%0], {%1, %2, %3, %4};" ::"r"(row_u + at), "r"(ou[0]), "r"(ou[1]), "r"(ou[2]), "r"(ou[3]) : "memory");
                }
                fence_async_shared();
                __syncwarp();
                if (!leader) {
                    if (lane == 0) mbar_arrive(half_done_bar(n));
                } else {
                    if (!mbar_wait(half_done_bar(n), (n >> 1) & 1u, abort_flag)) {
                        if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, STATUS_WAIT_EPILOGUE); }
                        gave_up = true;
                        break;
                    }
                    if (lane == 0) {
                        const int col = tile.n0 + c * 64, row = tile.row0 + quad * 32;
                        tma_store_2d(&p.map_a3, buffer(n), col, row);
                        tma_store_2d(&p.map_b3, buffer(n) + BOX_BYTES, col, row);
                        bulk_commit();
                    }
                }
                ++n;
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (CTAS == 2 && cta_rank) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
                else mbar_arrive(tempty_bar(acc));
            }
            ++iter;
        }
        if (leader && lane == 0) bulk_wait_all();   // shared memory stays until the last store has left it
        __syncwarp();
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int quad = warp & 3;         // TMEM lanes [32 * quad, 32 * quad + 32) belong to this warp
        const uint32_t stage = epi0 + (uint32_t)(warp - 2) * Config::EPI_WARP_BYTES;  // this warp's transpose buffer
        const int half = (warp - 2) >> 2;  // which half of the tile's columns this warp converts
        int iter = 0;
        for (int t = first_tile; t < total_tiles && !*abort_flag; t += tile_stride) {
            const Tile tile = decode_tile<MODE, B_MN, CTAS>(p, s_start, s_pair, s_order, t, cta_rank);
            if (!tile.valid) continue;
            const int acc = iter & 1;
            const uint32_t acc_phase = (uint32_t)(iter >> 1) & 1u;
            if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag)) {
                if (!*abort_flag) { *abort_flag = 1; atomicExch(p.status, STATUS_WAIT_EPILOGUE); }
                break;
            }
            tc_fence_after();
            const uint32_t taddr = tmem_base + ((uint32_t)(quad * 32) << 16) + (uint32_t)acc * BN;
            const long long row = (long long)tile.row0 + quad * 32 + lane;
            // Row-major pointers of this warp's 32 rows (row0w) for the coalesced paths: a warp moves a
            // 32-row x 32-column bf16 block as 8 rows x 64 contiguous bytes per instruction, transposing
            // between "one thread = one row" (the TMEM read layout) and that shape through shared memory.
            const long long row0w = (long long)tile.row0 + quad * 32;
            // 32-column chunks of this warp: its half of the tile's columns (4 of 8, or 2 of 4 in a narrow tile)
            const int c_begin = half * (tile.bn / 64), c_end = c_begin + tile.bn / 64;
            if (CTAS == 2 && !tile.rows_valid) {
                // second half of an odd pair-tile: these rows belong to nobody, nothing is stored
            } else if (MODE == MODE_SWIGLU) {
                __nv_bfloat16* G = (__nv_bfloat16*)p.out0 + row0w * p.ldc + tile.n0;
                __nv_bfloat16* U = (__nv_bfloat16*)p.out1 + row0w * p.ldc + tile.n0;
                __nv_bfloat16* H = (__nv_bfloat16*)p.out2 + row0w * p.ldc + tile.n0;
#pragma unroll 1
                for (int c = 2 * half; c < 2 * half + 2; ++c) {
                    uint32_t rg[32], ru[32];
                    tmem_ld32(taddr + c * 32, rg);
                    tmem_ld32(taddr + 128 + c * 32, ru);
                    tmem_ld_wait();
                    const int valid = p.N - (tile.n0 + c * 32);
                    if (valid >= 32) {
                        uint32_t wg[16], wu[16], wh[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) {
                            // G and U are stored as bf16 and H is computed from the stored values,
                            // so the backward (which re-reads G and U) sees exactly what H was built from
                            wg[j] = pack_bf16(__uint_as_float(rg[2 * j]), __uint_as_float(rg[2 * j + 1]));
                            wu[j] = pack_bf16(__uint_as_float(ru[2 * j]), __uint_as_float(ru[2 * j + 1]));
                            const float g0 = bf16_lo(wg[j]), g1 = bf16_hi(wg[j]);
                            wh[j] = pack_bf16(g0 * fast_sigmoid(g0) * bf16_lo(wu[j]), g1 * fast_sigmoid(g1) * bf16_hi(wu[j]));
                        }
                        store_block32(stage, lane, wg, G + c * 32, p.ldc);
                        store_block32(stage, lane, wu, U + c * 32, p.ldc);
                        store_block32(stage, lane, wh, H + c * 32, p.ldc);
                    } else if (valid > 0) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < valid) {
                                const __nv_bfloat16 gb = __float2bfloat16_rn(__uint_as_float(rg[i]));
                                const __nv_bfloat16 ub = __float2bfloat16_rn(__uint_as_float(ru[i]));
                                const float g = __bfloat162float(gb);
                                G[lane * p.ldc + c * 32 + i] = gb;
                                U[lane * p.ldc + c * 32 + i] = ub;
                                H[lane * p.ldc + c * 32 + i] = __float2bfloat16_rn(g * fast_sigmoid(g) * __bfloat162float(ub));
                            }
                    }
                }
            } else if (MODE == MODE_PLAIN) {
                __nv_bfloat16* C = (__nv_bfloat16*)p.out0 + row0w * p.ldc + tile.n0;
                __nv_bfloat16* remote = nullptr;  // scatter mode: where this lane's row goes (null: pad row)
                if (p.scatter_ret) {
                    const int index_in_expert = (int)row - s_start[tile.expert] * kRowPad;
                    if (index_in_expert < p.counts[tile.expert]) {
                        const int address = p.scatter_ret[row];
                        remote = (__nv_bfloat16*)p.scatter_base[address >> 26] + (long long)(address & ((1 << 26) - 1)) * p.ldc + tile.n0;
                    }
                }
                const bool wide = p.scatter_ret && p.scatter_wide && c_end - c_begin == 4 && p.N - (tile.n0 + c_begin * 32) >= 128;
                if (wide) {  // this warp's 128 columns are all there: scatter them as 256-byte row pieces
                    uint32_t w[64];
#pragma unroll
                    for (int cc = 0; cc < 4; ++cc) {
                        uint32_t r[32];
                        tmem_ld32(taddr + (c_begin + cc) * 32, r);
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            w[cc * 16 + j] = pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                    }
                    scatter_rows256(stage, lane, w, remote ? remote + c_begin * 32 : nullptr);
                }
#pragma unroll 1
                for (int c = wide ? c_end : c_begin; c < c_end; ++c) {
                    uint32_t r[32];
                    tmem_ld32(taddr + c * 32, r);
                    tmem_ld_wait();
                    const int valid = p.N - (tile.n0 + c * 32);
                    if (valid >= 32) {
                        uint32_t w[16];
#pragma unroll
                        for (int j = 0; j < 16; ++j) w[j] = pack_bf16(__uint_as_float(r[2 * j]), __uint_as_float(r[2 * j + 1]));
                        if (p.scatter_ret) scatter_block32(stage, lane, w, remote ? remote + c * 32 : nullptr);
                        else store_block32(stage, lane, w, C + c * 32, p.ldc);
                    } else if (valid > 0) {
                        float v[32];
#pragma unroll
                        for (int i = 0; i < 32; ++i) v[i] = __uint_as_float(r[i]);
                        if (!p.scatter_ret) store_row32_bf16(C + lane * p.ldc + c * 32, v, valid);
                        else if (remote) store_row32_bf16(remote + c * 32, v, valid);
                    }
                }
            } else if (MODE == MODE_ROUTER) {
                // scores = x . (W_hi + W_mid + W_lo)^T: the three partial products sit S columns apart
                float* C = (float*)p.out0 + row * p.ldc;
                const int S = p.group_stride;
#pragma unroll 1
                for (int c = half; c * 32 < S; c += 2) {
                    uint32_t r0[32], r1[32], r2[32];
                    tmem_ld32(taddr + c * 32, r0);
                    tmem_ld32(taddr + S + c * 32, r1);
                    tmem_ld32(taddr + 2 * S + c * 32, r2);
                    tmem_ld_wait();
                    const int valid = p.N - c * 32;
                    if (row < p.M) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < valid)
                                C[c * 32 + i] = (__uint_as_float(r2[i]) + __uint_as_float(r1[i])) + __uint_as_float(r0[i]);
                    }
                }
            } else if (MODE == MODE_WGRAD && ((p.transpose_out >> tile.problem) & 1)) {
                // the product is stored transposed, out[e][n][m] (row pitch M): the 32 lanes of a warp hold
                // consecutive m, so each store instruction writes one 128-byte line
                float* out = (float*)(tile.problem == 0 ? p.out0 : tile.problem == 1 ? p.out1 : p.out2);
                const long long ldc = p.M;
                float* C = out + (long long)tile.expert * p.c_slab + (long long)tile.n0 * ldc + row;
                const bool row_ok = row < p.M;
#pragma unroll 1
                for (int c = c_begin; c < c_end; ++c) {
                    uint32_t r[32];
                    tmem_ld32(taddr + c * 32, r);
                    tmem_ld_wait();
                    const int valid = p.N - (tile.n0 + c * 32);
                    if (row_ok) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < valid) C[(long long)(c * 32 + i) * ldc] = __uint_as_float(r[i]);
                    }
                }
            } else {
                float* out = (float*)(MODE != MODE_WGRAD || tile.problem == 0 ? p.out0 : tile.problem == 1 ? p.out1 : p.out2);
                float* C = out + (long long)tile.expert * p.c_slab + row * p.ldc + tile.n0;
                float* Cw = out + (long long)tile.expert * p.c_slab + row0w * p.ldc + tile.n0;  // this warp's first row
                const bool row_ok = row < p.M;  // WGRAD: rows of one expert's output; PLAIN_F32: rows of the single group
#pragma unroll 1
                for (int c = c_begin; c < c_end; ++c) {
                    uint32_t r[32];
                    tmem_ld32(taddr + c * 32, r);
                    tmem_ld_wait();
                    const int valid = p.N - (tile.n0 + c * 32);
                    if (valid >= 32) {
                        store_block32_f32(stage, lane, r, Cw + c * 32, p.ldc, (long long)p.M - row0w);
                    } else if (row_ok) {
#pragma unroll
                        for (int i = 0; i < 32; ++i)
                            if (i < valid) C[c * 32 + i] = __uint_as_float(r[i]);
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (CTAS == 2 && cta_rank) mbar_arrive_cluster(map_to_cta(tempty_bar(acc), 0));
                else mbar_arrive(tempty_bar(acc));
            }
            ++iter;
        }
        // rows stored into other GPUs' memory: one system-scope fence per thread after its last tile (the
        // kernel's completion orders them before whatever the stream signals next; a fence per tile only
        // made the accumulator wait for an NVLink round trip)
        if (MODE == MODE_PLAIN && p.scatter_ret) __threadfence_system();
    }

    // ------------------------------ teardown ---------------------------------------
    tc_fence_before();
    __syncthreads();
    if (s_abort) {
        // give copies and MMAs in flight a bounded time to land before shared memory and TMEM go away
        const unsigned long long start = global_ns();
        while (global_ns() - start < 2000000ull) __nanosleep(1000);
        __syncthreads();
    }
    // neither CTA of a pair may leave (or free tensor memory) while the other can still signal or read it
    if (CTAS == 2) cluster_sync();
    if (warp == 1) {
        tc_fence_after();
        if (CTAS == 2) asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
        else asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
    }
}

// ---- host side: tensor maps ------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    });
    return fn;
}

std::mutex g_map_mutex;
std::map<std::tuple<uint64_t, uint64_t, uint64_t, uint32_t, uint32_t>, CUtensorMap> g_maps;

// 2-D bf16 row-major matrix [outer, inner], box {64, box_outer}: 64 columns (128 bytes) with the 128-byte swizzle,
// for the operand tiles and for the epilogue boxes of dSwiGLU alike.
int make_map(CUtensorMap* out, uint64_t ptr, uint64_t inner, uint64_t outer, uint32_t box_outer, uint64_t pitch = 0) {
    constexpr uint32_t box_inner = 64;
    if (!pitch) pitch = inner;  // elements between consecutive rows
    auto key = std::make_tuple(ptr, inner | (pitch << 32), outer, box_inner, box_outer);
    {
        std::lock_guard<std::mutex> lock(g_map_mutex);
        auto it = g_maps.find(key);
        if (it != g_maps.end()) { *out = it->second; return 0; }
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return QMOE_ERR_STATE; }
    if (ptr & 15u) return fail_arg("tensor-core GEMM operand address must be 16-byte aligned");
    if ((pitch * 2) % 16) return fail_arg("tensor-core GEMM operand row pitch must be a multiple of 16 bytes");
    cuuint64_t dims[2] = {inner, outer};
    cuuint64_t strides[1] = {pitch * 2};
    cuuint32_t box[2] = {box_inner, box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, (void*)ptr, dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                     CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d (inner %llu, outer %llu, box %u x %u)", (int)rc,
                  (unsigned long long)inner, (unsigned long long)outer, box_inner, box_outer);
        return 999;
    }
    std::lock_guard<std::mutex> lock(g_map_mutex);
    if (g_maps.size() > 4096) g_maps.clear();
    g_maps[key] = *out;
    return 0;
}

}  // namespace

// 3-D bf16 tensor [outer][mid][inner] (dense), box {64, box_mid, 1}, 128-byte swizzle: the attention kernels' view of
// [batch][time][heads * 64], in which a box never crosses from one sequence into the next and positions past the end
// of a sequence arrive as zeros.
int make_map_3d(CUtensorMap* out, uint64_t ptr, uint64_t inner, uint64_t mid, uint64_t outer, uint32_t box_mid) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) { set_error("cuTensorMapEncodeTiled is not available from the driver"); return QMOE_ERR_STATE; }
    if (ptr & 15u) return fail_arg("tensor-core operand address must be 16-byte aligned");
    if ((inner * 2) % 16) return fail_arg("tensor-core operand row pitch must be a multiple of 16 bytes");
    cuuint64_t dims[3] = {inner, mid, outer};
    cuuint64_t strides[2] = {inner * 2, inner * mid * 2};
    cuuint32_t box[3] = {64, box_mid, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult rc = fn(out, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, (void*)ptr, dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (rc != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d (3-D: inner %llu, mid %llu, outer %llu)", (int)rc,
                  (unsigned long long)inner, (unsigned long long)mid, (unsigned long long)outer);
        return 999;
    }
    return 0;
}

namespace {

template <int MODE, bool A_MN, bool B_MN, int CTAS = 1>
int launch(const GemmParams& p, cudaStream_t stream) {
    static int grid_of[64] = {0};  // per device: blocks to launch (0: not configured yet)
    constexpr int SMEM_BYTES = Cfg<CTAS, MODE>::SMEM_BYTES;
    // a block has 227 KiB, its static tables included: two or three of (kMaxExperts + 1) ints plus two words
    static_assert(SMEM_BYTES + (starts_in_shared<MODE, CTAS>() ? 3 : 1) * 4 * (kMaxExperts + 1) + 16 <= 227 * 1024,
                  "operand ring + epilogue staging + tables exceed the shared memory of a block");
    int dev = 0;
    QMOE_CUDA(cudaGetDevice(&dev));
    if (dev >= 64) return fail_arg("device ordinal beyond 63");
    auto kernel = grouped_gemm_kernel<MODE, A_MN, B_MN, CTAS>;
    cudaLaunchConfig_t config = {};
    cudaLaunchAttribute attribute[1];
    config.blockDim = dim3(NUM_THREADS);
    config.dynamicSmemBytes = SMEM_BYTES;
    config.stream = stream;
    if (CTAS == 2) {
        attribute[0].id = cudaLaunchAttributeClusterDimension;
        attribute[0].val.clusterDim.x = 2;
        attribute[0].val.clusterDim.y = 1;
        attribute[0].val.clusterDim.z = 1;
        config.attrs = attribute;
        config.numAttrs = 1;
    }
    if (!grid_of[dev]) {
        QMOE_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES));
        int grid = sm_count();
        if (CTAS == 2) {
            // a persistent grid: launch exactly as many pairs as can be resident together (a GPC with an
            // odd number of usable SMs leaves one without a partner)
            int clusters = 0;
            config.gridDim = dim3((unsigned)(grid & ~1));
            QMOE_CUDA(cudaOccupancyMaxActiveClusters(&clusters, kernel, &config));
            if (clusters < 1) { set_error("no CTA pair of the tensor-core GEMM fits on this device"); return QMOE_ERR_STATE; }
            grid = 2 * (clusters < grid / 2 ? clusters : grid / 2);
        }
        grid_of[dev] = grid;
    }
    config.gridDim = dim3((unsigned)grid_of[dev]);
    QMOE_CUDA(cudaLaunchKernelEx(&config, kernel, p));
    count_tensor_core_launch();
    QMOE_LAUNCH_CHECK("grouped_gemm_kernel");
    return 0;
}

// CTAs per output tile of the expert GEMMs: 2 (a CTA pair per 256 x 256 tile); the one-CTA kernel
// (128 x 256 tiles) stays reachable for the parity tests through qmoe_test_select_variant.
int gemm_ctas() { return kernel_variant(QMOE_VARIANT_SINGLE_CTA_GEMM) ? 1 : 2; }

}  // namespace

bool tcgen05_shape_ok(long long width, long long hidden) { return width % 8 == 0 && hidden % 8 == 0 && width >= 8 && hidden >= 8; }

// G, U, H [rows, h] = SwiGLU(X [rows, d]; Wg, Wu [E*h, d])
int tc_swiglu_forward(const qmoe_route_t* r, const qmoe_experts_t* ex, uint64_t x, uint64_t g, uint64_t u, uint64_t h,
                      cudaStream_t stream) {
    GemmParams p = {};
    const uint64_t rows = (uint64_t)r->rows_bound, d = (uint64_t)ex->width, hd = (uint64_t)ex->hidden, E = (uint64_t)ex->experts;
    if (int rc = make_map(&p.map_a, x, d, rows, BM)) return rc;
    if (int rc = make_map(&p.map_b, ex->w_gate, d, E * hd, 128)) return rc;
    if (int rc = make_map(&p.map_b2, ex->w_up, d, E * hd, 128)) return rc;
    p.map_a2 = p.map_a;
    p.offsets = (const int*)r->offsets; p.counts = (const int*)r->counts; p.status = device_status_address();
    p.out0 = (void*)g; p.out1 = (void*)u; p.out2 = (void*)h;
    p.ldc = (long long)hd; p.experts = ex->experts; p.n_tiles = ceil_div((long long)hd, 128);
    p.N = (int)hd; p.K = (int)d; p.b_rows = (int)hd; p.segments = 1;
    if (gemm_ctas() == 2) return launch<MODE_SWIGLU, false, false, 2>(p, stream);
    return launch<MODE_SWIGLU, false, false>(p, stream);
}

// C [rows, N] = A [rows, K] . B_e^T with B stacked [E*N, K]
void set_scatter(GemmParams& p, const TcScatter* scatter) {
    if (!scatter) return;
    p.scatter_ret = scatter->ret;
    p.scatter_wide = !kernel_variant(QMOE_VARIANT_NARROW_SCATTER);
    for (int i = 0; i < 16; ++i) p.scatter_base[i] = scatter->base[i];
}

int tc_rows_nt(const qmoe_route_t* r, int experts, uint64_t a, uint64_t b, uint64_t c, long long K, long long N,
               cudaStream_t stream, const TcScatter* scatter) {
    GemmParams p = {};
    set_scatter(p, scatter);
    if (int rc = make_map(&p.map_a, a, (uint64_t)K, (uint64_t)r->rows_bound, BM)) return rc;
    const int ctas = gemm_ctas();
    if (int rc = make_map(&p.map_b, b, (uint64_t)K, (uint64_t)experts * N, BN / ctas)) return rc;
    p.map_a2 = p.map_a; p.map_b2 = p.map_b;
    p.offsets = (const int*)r->offsets; p.counts = (const int*)r->counts; p.status = device_status_address();
    p.out0 = (void*)c; p.ldc = N; p.experts = experts; p.n_tiles = ceil_div(N, BN);
    p.N = (int)N; p.K = (int)K; p.b_rows = (int)N; p.segments = 1;
    if (ctas == 2) return launch<MODE_PLAIN, false, false, 2>(p, stream);
    return launch<MODE_PLAIN, false, false>(p, stream);
}

// C [rows, N] = A [rows, K] . B_e (+ A2 . B2_e) with B stacked [E*K, N]
int tc_rows_nn(const qmoe_route_t* r, int experts, uint64_t a, uint64_t b, uint64_t a2, uint64_t b2, uint64_t c,
               long long K, long long N, cudaStream_t stream, const TcScatter* scatter) {
    GemmParams p = {};
    set_scatter(p, scatter);
    if (int rc = make_map(&p.map_a, a, (uint64_t)K, (uint64_t)r->rows_bound, BM)) return rc;
    if (int rc = make_map(&p.map_b, b, (uint64_t)N, (uint64_t)experts * K, 64)) return rc;
    p.map_a2 = p.map_a; p.map_b2 = p.map_b;
    p.segments = 1;
    if (a2) {
        if (int rc = make_map(&p.map_a2, a2, (uint64_t)K, (uint64_t)r->rows_bound, BM)) return rc;
        if (int rc = make_map(&p.map_b2, b2, (uint64_t)N, (uint64_t)experts * K, 64)) return rc;
        p.segments = 2;
    }
    p.offsets = (const int*)r->offsets; p.counts = (const int*)r->counts; p.status = device_status_address();
    p.out0 = (void*)c; p.ldc = N; p.experts = experts; p.n_tiles = ceil_div(N, BN);
    p.N = (int)N; p.K = (int)K; p.b_rows = (int)K;
    if (gemm_ctas() == 2) return launch<MODE_PLAIN, false, true, 2>(p, stream);
    return launch<MODE_PLAIN, false, true>(p, stream);
}

// dG, dU [rows, h] from dY [rows, d], Wd stacked [E*d, h] and the saved G, U: the product dH = dY . Wd_e
// only ever lives in tensor memory
int tc_dswiglu(const qmoe_route_t* r, int experts, uint64_t dy, uint64_t w_down, uint64_t g, uint64_t u, uint64_t dg,
               uint64_t du, long long d, long long h, cudaStream_t stream) {
    GemmParams p = {};
    if (int rc = make_map(&p.map_a, dy, (uint64_t)d, (uint64_t)r->rows_bound, BM)) return rc;
    if (int rc = make_map(&p.map_b, w_down, (uint64_t)h, (uint64_t)experts * d, 64)) return rc;
    // the epilogue's boxes: G and U in, dG and dU out, 32 rows x 32 columns each
    const uint64_t rows = (uint64_t)r->rows_bound;
    if (int rc = make_map(&p.map_a2, g, (uint64_t)h, rows, 32)) return rc;
    if (int rc = make_map(&p.map_b2, u, (uint64_t)h, rows, 32)) return rc;
    if (int rc = make_map(&p.map_a3, dg, (uint64_t)h, rows, 32)) return rc;
    if (int rc = make_map(&p.map_b3, du, (uint64_t)h, rows, 32)) return rc;
    p.offsets = (const int*)r->offsets; p.counts = (const int*)r->counts; p.status = device_status_address();
    p.out0 = (void*)dg; p.out1 = (void*)du; p.in0 = (const void*)g; p.in1 = (const void*)u;
    p.ldc = h; p.experts = experts; p.n_tiles = ceil_div(h, BN);
    p.N = (int)h; p.K = (int)d; p.b_rows = (int)d; p.segments = 1;
    if (gemm_ctas() == 2) return launch<MODE_DSWIGLU, false, true, 2>(p, stream);
    return launch<MODE_DSWIGLU, false, true>(p, stream);
}

// scores [T, E] (fp32) = x [T, d] . (W_hi + W_mid + W_lo)^T, w3 = [3S, d] bf16 with the three terms S rows apart
int tc_router_forward(uint64_t x, uint64_t w3, uint64_t scores, long long T, long long d, int E, int S, cudaStream_t stream) {
    GemmParams p = {};
    if (int rc = make_map(&p.map_a, x, (uint64_t)d, (uint64_t)T, BM)) return rc;
    if (int rc = make_map(&p.map_b, w3, (uint64_t)d, (uint64_t)3 * S, BN)) return rc;
    p.map_a2 = p.map_a; p.map_b2 = p.map_b;
    p.status = device_status_address();
    p.out0 = (void*)scores; p.ldc = E; p.experts = 1; p.n_tiles = 1;
    p.M = (int)T; p.N = E; p.K = (int)d; p.b_rows = 0; p.segments = 1; p.plain_rows = (int)T; p.group_stride = S;
    return launch<MODE_ROUTER, false, false>(p, stream);
}

// C [T, N] (fp32) = A [T, K] . B [K, N] (one group, rows masked at T)
int tc_plain_f32_nn(uint64_t a, uint64_t b, uint64_t c, long long T, long long K, long long N, cudaStream_t stream) {
    GemmParams p = {};
    if (int rc = make_map(&p.map_a, a, (uint64_t)K, (uint64_t)T, BM)) return rc;
    if (int rc = make_map(&p.map_b, b, (uint64_t)N, (uint64_t)K, 64)) return rc;
    p.map_a2 = p.map_a; p.map_b2 = p.map_b;
    if (c & 15u || (N * 4) % 16) return fail_arg("fp32 output must be 16-byte aligned with a 16-byte row pitch");
    p.status = device_status_address();
    p.out0 = (void*)c; p.ldc = N; p.c_slab = 0; p.experts = 1; p.n_tiles = ceil_div(N, BN);
    p.M = (int)T; p.N = (int)N; p.K = (int)K; p.b_rows = 0; p.segments = 1; p.plain_rows = (int)T;
    return launch<MODE_PLAIN_F32, false, true>(p, stream);
}

// partial[s] [M, N] (fp32) = A[rows of split s]^T . B[rows of split s]; A [T, M] with row pitch a_pitch, B [T, N]
int tc_split_wgrad(uint64_t a, long long a_pitch, uint64_t b, uint64_t partial, const int* offsets, const int* counts,
                   int splits, long long T, long long M, long long N, cudaStream_t stream) {
    GemmParams p = {};
    if (int rc = make_map(&p.map_a, a, (uint64_t)M, (uint64_t)T, 64, (uint64_t)a_pitch)) return rc;
    if (int rc = make_map(&p.map_b, b, (uint64_t)N, (uint64_t)T, 64)) return rc;
    p.map_a2 = p.map_a; p.map_b2 = p.map_b;
    if (partial & 15u || (N * 4) % 16) return fail_arg("fp32 output must be 16-byte aligned with a 16-byte row pitch");
    p.offsets = offsets; p.counts = counts; p.status = device_status_address();
    p.out0 = (void*)partial; p.ldc = N; p.c_slab = M * N; p.experts = splits;
    p.m_tiles = ceil_div(M, BM); p.n_tiles = ceil_div(N, BN);
    p.M = (int)M; p.N = (int)N; p.K = 0; p.segments = 1; p.problems = 1;
    return launch<MODE_WGRAD, true, true>(p, stream);
}

// The three weight gradients of an expert FFN in one launch (one tile queue: fewer, fuller rounds of the
// persistent grid than three launches, and dWg / dWu tiles that share the layer input run side by side):
// dWd [d, h] = dY^T . H, dWg [h, d] = dG^T . X, dWu [h, d] = dU^T . X per expert, fp32, the contraction running
// over the expert's dispatched rows.  Tiles are 128 * ctas rows x 256 (or a last 128) columns, so all three
// run in the orientation (rows x columns = d x h or h x d) that leaves less padding; those stored the other
// way round are written transposed.
int tc_wgrad3(const qmoe_route_t* r, int experts, uint64_t dy, uint64_t h_act, uint64_t x, uint64_t dg, uint64_t du,
              uint64_t d_w_down, uint64_t d_w_gate, uint64_t d_w_up, long long d, long long h, cudaStream_t stream) {
    GemmParams p = {};
    if ((d_w_down | d_w_gate | d_w_up) & 15u || (d * 4) % 16 || (h * 4) % 16)
        return fail_arg("weight-gradient output must be 16-byte aligned with a 16-byte row pitch");
    const int ctas = gemm_ctas();
    auto padded = [&](long long m, long long n) { return ceil_div(m, BM * ctas) * (BM * ctas) * ceil_div(n, BN / 2) * (BN / 2); };
    const bool rows_are_d = padded(d, h) <= padded(h, d);
    const long long m = rows_are_d ? d : h, n = rows_are_d ? h : d;
    const uint64_t rows = (uint64_t)r->rows_bound;
    // kernel A = the operand with m columns, B = the one with n columns
    const uint64_t a_of[3] = {rows_are_d ? dy : h_act, rows_are_d ? x : dg, rows_are_d ? x : du};
    const uint64_t b_of[3] = {rows_are_d ? h_act : dy, rows_are_d ? dg : x, rows_are_d ? du : x};
    CUtensorMap* ma[3] = {&p.map_a, &p.map_a2, &p.map_a3};
    CUtensorMap* mb[3] = {&p.map_b, &p.map_b2, &p.map_b3};
    for (int i = 0; i < 3; ++i) {
        if (int rc = make_map(ma[i], a_of[i], (uint64_t)m, rows, 64)) return rc;
        if (int rc = make_map(mb[i], b_of[i], (uint64_t)n, rows, 64)) return rc;
    }
    p.offsets = (const int*)r->offsets; p.counts = (const int*)r->counts; p.status = device_status_address();
    p.out0 = (void*)d_w_down; p.out1 = (void*)d_w_gate; p.out2 = (void*)d_w_up;
    // dWd is [d, h]: natural when the kernel's rows are d; dWg, dWu are [h, d]: natural when they are h
    p.transpose_out = rows_are_d ? 0b110 : 0b001;
    p.ldc = n; p.c_slab = d * h; p.experts = experts; p.problems = 3;
    p.m_tiles = ceil_div(m, BM * ctas); p.n_tiles = ceil_div(n, BN);
    p.M = (int)m; p.N = (int)n; p.K = 0; p.segments = 1;
    if (kernel_variant(QMOE_VARIANT_WGRAD_PER_PRODUCT)) {  // one launch per product, for comparison
        void* const outs[3] = {p.out0, p.out1, p.out2};
        const int transposed = p.transpose_out;
        for (int i = 0; i < 3; ++i) {
            GemmParams q = p;
            q.map_a = *ma[i]; q.map_b = *mb[i]; q.out0 = outs[i]; q.transpose_out = (transposed >> i) & 1; q.problems = 1;
            if (int rc = ctas == 2 ? launch<MODE_WGRAD, true, true, 2>(q, stream) : launch<MODE_WGRAD, true, true>(q, stream)) return rc;
        }
        return 0;
    }
    if (ctas == 2) return launch<MODE_WGRAD, true, true, 2>(p, stream);
    return launch<MODE_WGRAD, true, true>(p, stream);
}

// out [M, N] (fp32) = A^T . B over the rows of ONE group (counts[0] rows from row offsets[0]): A [rows, M], B [rows, N].
// The weight gradient of a plain linear map (the language-model head), on CTA pairs.  With `groups` > 1 the rows are cut
// into that many ranges (offsets[g], counts[g]; every offset a multiple of 128) and range g leaves its own product in
// out + g * slab: a short, wide product then fills the machine, and the caller adds the slabs in a fixed order.
int tc_wgrad1(const qmoe_route_t* r, uint64_t a, uint64_t b, uint64_t out, long long M, long long N, cudaStream_t stream,
              int groups, long long slab) {
    GemmParams p = {};
    if (out & 15u || (N * 4) % 16) return fail_arg("weight-gradient output must be 16-byte aligned with a 16-byte row pitch");
    const int ctas = gemm_ctas();
    const uint64_t rows = (uint64_t)r->rows_bound;
    if (int rc = make_map(&p.map_a, a, (uint64_t)M, rows, 64)) return rc;
    if (int rc = make_map(&p.map_b, b, (uint64_t)N, rows, 64)) return rc;
    p.map_a2 = p.map_a; p.map_b2 = p.map_b; p.map_a3 = p.map_a; p.map_b3 = p.map_b;
    p.offsets = (const int*)r->offsets; p.counts = (const int*)r->counts; p.status = device_status_address();
    p.out0 = (void*)out; p.ldc = N; p.c_slab = slab; p.experts = groups; p.problems = 1;
    p.m_tiles = ceil_div(M, BM * ctas); p.n_tiles = ceil_div(N, BN);
    p.M = (int)M; p.N = (int)N; p.K = 0; p.segments = 1;
    if (ctas == 2) return launch<MODE_WGRAD, true, true, 2>(p, stream);
    return launch<MODE_WGRAD, true, true>(p, stream);
}

}  // namespace qmoe
