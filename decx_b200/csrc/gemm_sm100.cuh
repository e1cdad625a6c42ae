// Persistent, warp-specialised tcgen05 GEMM for sm_100a.
//
//   D(M x N) = alpha * A(M x K) * B(K x N) + beta * C(M x N)         row-major, pitched
//
// replaces the SIMT kernels behind de::blas::cuda::GEMM
// (srcs/modules/BLAS/GEMM/CUDA/large_squares/{fp32,fp16,64b}/*_kernels.cu in the
// reference: 256-thread CTAs, one shared-memory stage, FMA inner loop) with:
//
//   warp 0      TMA producer: 128-byte-swizzled tiles of A (K-major) and of row-major
//               B (consumed MN-major, so B is never transposed) into a ring of stages
//   warp 1      allocates TMEM and issues tcgen05.mma; fp32 accumulators live in TMEM,
//               two of them, so draining one overlaps the MMAs into the other
//   warps 2..   epilogue: tcgen05.ld -> alpha/beta/C -> a 32-row x 128-byte staging tile per warp in
//               shared memory -> TMA bulk store (rows past M dropped by the hardware); predicated
//               per-thread stores where D's rows are not 16-byte aligned or an N edge is ragged
//
// The CTAs are persistent (one per SM) and walk a rasterised tile list; a soft, time-limited barrier
// between tile rounds keeps them at the same K position so that shared A/B slabs hit in L2
// (g_wave_ticket).  Optionally B arrives while the kernel runs, in column panels guarded by flags
// (GemmParams::panel_flags): the tile list is then ordered panel by panel.
//
// Accumulation chains.  The tensor core adds into its fp32 accumulator with truncation, so a
// long chain of same-signed terms drifts by about (chain length) * 2^-24 relative -- 4e-6 at
// K = 1000 on all-positive data, beyond fp32 behaviour.  The 3xTF32 kernel therefore
// accumulates in TMEM only over chunks of CHUNK_KB k-blocks (K = 128); its eight epilogue
// warps add every finished chunk into fp32 registers (round to nearest) while the MMAs of
// the next chunk run into the other TMEM accumulator.  The fp16 kernel keeps one chain per
// tile: its output precision (2^-11) is far coarser than the drift.
//
// KIND 0  fp16 operands, kind::f16, fp16 output.
// KIND 1  fp32 operands pre-split into tf32 (hi, lo) planes, kind::tf32, three MMAs per
//         K step (lo*hi, hi*lo, hi*hi) into one accumulator = "3xTF32"; fp32 output.
//         Interleaved complex problems arrive here as a real problem of twice the K and
//         N extents (see prepass.cuh), only the epilogue knows about (re, im) pairs.
// CTAS 1  one CTA per 128 x 256 tile.
// CTAS 2  a CTA pair (cluster of 2) per 256 x 256 tile, tcgen05 cta_group::2: each CTA
//         loads its own 128 rows of A and its own 128 columns of B (no multicast), the
//         pair's leader issues the MMAs, each CTA keeps its 128 x 256 accumulator rows.
//
// NACC 2  (fp16 pairs only) the pair computes 256 x 512: two accumulators share every A tile, which
//         cuts the operand traffic from L2 from 64 to 48 bytes per clock and SM -- the 256 x 256 tile
//         sits at ~70 % of what the L2 can deliver without multicast and stalls on it.  CTA r loads
//         the contiguous columns [512 t + 256 r, +256); accumulator h multiplies columns
//         [.. + 128 h, +128) of both CTAs.  Both TMEM accumulators belong to one tile, so the epilogue
//         (eight warps, four per accumulator) no longer overlaps the next tile's MMAs: used for long K.
//
// FETCH f (fp16 pairs, row-sharded multi-GPU GEMM) adds f "courier" warps per CTA that bring B into this GPU's
//         memory WHILE the tiles are computed: they walk a job list (source address in a peer GPU's memory,
//         rows, column range, an optional gate word), copy 8 KB batches with 16-byte peer loads and local
//         stores, count the batches per column panel and raise that panel's flag when it is complete -- the flag
//         the TMA producer waits on.  Pieces this GPU is the first holder of are "published" through a second
//         flag that the other GPUs' couriers gate on, so one kernel per GPU does scatter + all-gather of B,
//         the product and (through D in the owner's memory) the gather.  All TMA loads still read local memory.
//
// Ragged M/N/K: tensor maps carry the logical extents, so out-of-range parts of a box
// are zero-filled by TMA on loads and dropped on stores.  No host-side padding.
// Every wait is bounded: on time-out the role writes a code to *status and unwinds.
#pragma once
#include <cuda_fp16.h>
#include "sm100_ptx.cuh"

namespace dxb {

enum EpilogueMode : int { EPI_REAL = 0, EPI_COMPLEX = 1 };

// status codes written by the kernel (0 = ok)
enum KernelStatus : unsigned {
    KS_OK = 0,
    KS_TIMEOUT_PRODUCER = 0x101,
    KS_TIMEOUT_MMA_FULL = 0x102,
    KS_TIMEOUT_MMA_ACC = 0x103,
    KS_TIMEOUT_EPILOGUE = 0x104,
    KS_TIMEOUT_TAIL = 0x105,
    KS_TIMEOUT_PANEL = 0x106,
    KS_TIMEOUT_FETCH = 0x107,
};
constexpr int MAX_PANELS = 16;

struct GemmParams {
    uint32_t M, N, K;          // real problem extents seen by the MMA (complex: N, K doubled)
    void* D;                   // fp16 (KIND 0) or fp32 (KIND 1)
    const void* C;             // same type as D, or nullptr
    uint64_t ldd, ldc;         // in scalars of the output type
    float alpha_re, alpha_im, beta_re, beta_im;
    int epi_mode;              // EpilogueMode
    int vec_d, vec_c;          // 1 if 16-byte vector access to D / C rows is legal
    int d_tma;                 // 1: D is written by TMA bulk stores from a shared-memory staging tile (128-byte rows,
                               //    edges clipped in hardware); 0: predicated per-thread stores
    int c_tma;                 // 1 (needs d_tma): boxes of C are brought into the staging tile by TMA loads (tmC)
    int b_chunked_map;         // 1: the B maps are 3-D (column, k, 128-byte chunk): one TMA fetches a whole stage
                               // 0: 2-D maps, one TMA per 128-byte column chunk
    uint32_t tiles_m, tiles_n; // in units of (128*CTAS) x 256
    uint32_t group_m;          // rasterisation group height, in tiles
    unsigned* status;          // device word, may be nullptr
    unsigned long long wait_limit_ns;
    // Column panels of B that arrive while the kernel runs (row-sharded multi-GPU GEMM): tiles are walked panel
    // by panel, and before a producer loads its first tile of panel i it waits (bounded) until
    // panel_flags[i] has reached panel_epoch -- written, after the panel's data, by the stream that delivers B.
    // n_panels == 1 and panel_flags == nullptr for an ordinary GEMM.
    uint32_t n_panels;
    uint32_t panel_end[MAX_PANELS];   // exclusive end of each panel, in tile columns
    const unsigned* panel_flags;
    unsigned panel_epoch;
    // soft lockstep of the persistent CTAs (see g_wave_ticket)
    unsigned sync_base;        // value of the ticket counter when this launch starts
    unsigned sync_on;          // 0 = off
    unsigned sync_limit_ns;    // how long a producer waits for the others before it goes on alone
    // optional timing record (device memory, zeroed by the host; nullptr = off), in ns of %globaltimer:
    //   [0..15] when panel i was complete (couriers), [16] start of CTA 0, [17] latest CTA end,
    //   [18] sum over the loaders of the time spent waiting for panel flags, [19] number of such waits,
    //   [20] sum over the MMA threads of the time spent waiting for operands (full barriers), [21] ... for a free
    //   accumulator, [22] ... of their whole tile loops, [23] number of MMA threads counted
    unsigned long long* stats;
    // Implicit-GEMM convolution (3xTF32 kernels; conv_tw == 0: an ordinary GEMM).  The 128 rows of
    // an M tile are a conv_tw x (128 / conv_tw) rectangle of output positions, row r = (r / conv_tw, r % conv_tw);
    // tile index (tm * CTAS + rank of the CTA in its pair) = ty * conv_tiles_x + tx.  The A maps are 4-D views of the zero-bordered source planes,
    // (k within a kernel row, x, kernel row i, y): k-block kb is kernel row kb / conv_kbi, floats
    // [32 * (kb % conv_kbi), +32) of its kw * C contiguous floats.  The D map is 3-D (kernel, x, y).
    uint32_t conv_tw, conv_tiles_x, conv_kbi;
};

// One piece of B a courier warp copies: rows [row0, row0 + rows) x bytes [byte0, byte0 + bytes) of every row, from
// `src` to `dst` (both laid out like the replica, same row pitch).  Two directions:
//   pull  (dst == nullptr: this GPU's replica; src usually another GPU's memory): the piece counts towards the
//         panel's "complete here" flag; with `publish` it also counts towards this GPU's publish flag.
//   push  (dst = another GPU's replica, src local): when the whole job is stored, `notify` -- a word in the TARGET's
//         memory, its publish flag for the panel -- is set to the epoch.  Stores over NVLink are posted: no
//         request has to travel towards the sender, whose inbound link may be busy receiving D.
//         With publish == FETCH_MULTICAST both `dst` and `notify` are addresses in an NVLink multicast mapping of
//         the replicas and their flags: every store is replicated by the switch into all bound GPUs, so the owner
//         sends B over its link ONCE and no GPU has to fetch pieces from another.
// rows == 0 is a piece something else delivers (a pushing GPU, a copy engine): the courier only waits for its gate
// and counts it.
struct FetchJob {
    const uint8_t* src;
    const unsigned* gate;      // word that must have reached `epoch` before src may be read; nullptr: readable now
    uint8_t* dst;              // nullptr: the local replica
    unsigned* notify;          // push jobs: word (in the target's memory) to set when the job is complete
    uint32_t row0, rows;
    uint32_t byte0, bytes;     // bytes % 16 == 0
    uint32_t panel;            // column panel the piece belongs to
    uint32_t publish;          // pull jobs: 1 = other GPUs fetch this piece from here once it has landed (pub_flags);
                               // push jobs: FETCH_MULTICAST = dst / notify are multicast addresses
};
constexpr uint32_t FETCH_MULTICAST = 2;
constexpr uint32_t FETCH_UNROLL = 16;                   // 512-byte segments per batch (one warp, one go): 8 KB
__host__ __device__ inline uint32_t fetch_job_batches(uint32_t rows, uint32_t bytes) {
    const uint64_t segs = uint64_t(rows) * ((bytes + 511u) / 512u);
    return segs == 0 ? 1u : uint32_t((segs + FETCH_UNROLL - 1) / FETCH_UNROLL);
}
struct FetchParams {
    const FetchJob* jobs;      // device memory
    uint32_t n_jobs;
    uint32_t total_batches;    // sum of fetch_job_batches over the jobs
    uint8_t* dst;              // this GPU's replica of B
    uint64_t pitch;            // bytes per row, source and destination
    unsigned* arrived;         // [MAX_PANELS] batches stored so far, zero at launch
    unsigned* published;       // [MAX_PANELS] batches of publishing jobs stored so far, zero at launch
    unsigned* next_batch;      // the next batch nobody has taken yet, zero at launch
    unsigned* job_done;        // [n_jobs] batches stored per job (push jobs), zero at launch
    unsigned* ready_flags;     // [MAX_PANELS] <- epoch when every batch of the panel is stored (= GemmParams::panel_flags)
    unsigned* pub_flags;       // [MAX_PANELS] <- epoch when every publishing batch of the panel is stored
    unsigned epoch;
    uint32_t need[MAX_PANELS];       // batches per panel
    uint32_t pub_need[MAX_PANELS];   // publishing batches per panel (0: nothing to publish)
    // D forwarding (256 x 512 tiles only; nullptr: the epilogue stores D directly).  When D lives in another GPU's
    // memory, every CTA of every GPU finishes its tile at about the same time and the TMA stores of all of them hit
    // one NVLink port as a burst; the accumulators are released only when the last box has left shared memory, so
    // the burst delays the next tile's MMAs (measured: 6 % on the sender, 9 % on the receiver whose own epilogue
    // collides with it).  With a stage the epilogue stores its part of the tile into a ring of two tiles per CTA in
    // LOCAL memory (it stays in L2), and the courier warps copy it to D with plain 16-byte stores while the next
    // tile is being multiplied.  Layout: CTA b, ring slot s, row r: fwd_stage + ((b * 2 + s) * 128 + r) * 1024 bytes.
    uint8_t* fwd_stage;
    uint64_t fwd_stage_bytes;        // host side only: size of the ring area
};

// Ticket counter of the soft tile barrier.  All CTAs of a launch are resident at once (one per SM), and
// they share A row slabs and B column slabs through L2 only while they walk K at the same pace; left
// alone they drift apart and the slabs are fetched from HBM again and again.  So before a producer
// starts loading its next tile it takes a ticket and waits -- for a bounded time, then it carries on
// regardless -- until every worker has finished issuing its previous tile.  The barrier is a hint:
// releasing early or late changes DRAM traffic, never results.  Every launch adds exactly n_tiles
// tickets, so the host can hand each launch its starting value.
__device__ unsigned g_wave_ticket;


template <int KIND, int CTAS, int NACC = 1, int FETCH = 0, int BNV = 256>
struct GemmCfg {
    static_assert(BNV == 256 || (BNV == 64 && KIND == 1 && CTAS == 1) || (BNV == 128 && KIND == 1),
                  "narrow accumulators: 3xTF32 only (64 columns: single-CTA tiles)");
    static_assert(NACC == 1 || (NACC == 2 && KIND == 0 && CTAS == 2), "two accumulators per tile: fp16 CTA pairs only");
    static_assert(FETCH == 0 || (KIND == 0 && CTAS == 2), "courier warps: fp16 CTA pairs only");
    static constexpr int ELEM = (KIND == 0) ? 2 : 4;
    static constexpr int NPL = (KIND == 0) ? 1 : 2;       // operand planes (hi, lo)
    static constexpr int BM = 128;                        // rows per CTA
    static constexpr int BN = BNV;                        // UMMA N = columns of one accumulator (64, 128: small problems, few kernels)
    static constexpr int BN_TILE = BN * NACC;             // columns of one tile (NACC accumulators share each A tile)
    static constexpr int BN_LOAD = BN_TILE / CTAS;        // columns of B this CTA loads per stage
    static constexpr int BK = 128 / ELEM;                 // one 128-byte swizzle row of K
    static constexpr int UMMA_K = 32 / ELEM;
    static constexpr int CHUNK_N = 128 / ELEM;            // B columns per 128-byte row
    static constexpr int B_CHUNKS = BN_LOAD / CHUNK_N;
    static constexpr int A_TILE = BM * 128;               // bytes per plane
    static constexpr int B_CHUNK_BYTES = BK * 128;
    static constexpr int B_TILE = B_CHUNKS * B_CHUNK_BYTES;
    static constexpr int STAGE = NPL * (A_TILE + B_TILE);
    static constexpr int STAGES = (192 * 1024) / STAGE;
    static constexpr int TMEM_COLS = 512;                 // two 256-column accumulators
    static constexpr bool PROMOTE = (KIND == 1);          // chunked TMEM chains summed in registers
    static constexpr int CHUNK_KB = 4;                    // k-blocks per TMEM chain when PROMOTE
    static constexpr int EPI_WARPS = PROMOTE ? 8 : 4 * NACC;
    static constexpr int EPI_COLS = PROMOTE ? BN / 2 : BN;   // accumulator columns per epilogue thread
    static constexpr int ACC_ARRIVALS = (EPI_WARPS / NACC) * CTAS;   // epilogue warps (of the pair) per accumulator
    static constexpr int THREADS = 64 + 32 * EPI_WARPS + 32 * FETCH;
    static constexpr int STAGING = EPI_WARPS * 4096;      // per epilogue warp: 32 rows x 128 bytes of output
    static constexpr int MAILBOX = (FETCH > 0) ? 64 : 0;  // D forwarding: parts published / forwarded per epilogue warp
    static constexpr int SMEM_BYTES = STAGES * STAGE + STAGING + 1024 /*alignment slack*/ + 256 /*barriers*/ + MAILBOX;
    static_assert(16 * STAGES + 32 + 8 + 16 + 8 * EPI_WARPS <= 256, "barrier area");
    static constexpr uint32_t IDESC = umma_idesc(KIND == 0 ? 0u : 2u, false, true, BM * CTAS, BN);
};

// tile index -> (tile_m, tile_n), walking groups of `group_m` tile rows column by column
// so that the CTAs running at one time share a small set of A rows and B columns in L2.
// Panels (see GemmParams) are the outermost level: all tiles of panel 0 come first.  Returns the panel index.
__device__ __forceinline__ uint32_t tile_coords(uint32_t t, const GemmParams& p, uint32_t& tm, uint32_t& tn) {
    uint32_t begin = 0, pi = 0;
    for (;; ++pi) {
        const uint32_t cnt = p.tiles_m * (p.panel_end[pi] - begin);
        if (t < cnt || pi + 1 >= p.n_panels) break;
        t -= cnt;
        begin = p.panel_end[pi];
    }
    const uint32_t width = p.panel_end[pi] - begin;
    const uint32_t per_group = p.group_m * width;
    const uint32_t g = t / per_group;
    const uint32_t first_m = g * p.group_m;
    const uint32_t rows = min(p.group_m, p.tiles_m - first_m);
    const uint32_t r = t - g * per_group;
    tm = first_m + r % rows;
    tn = begin + r / rows;
    return pi;
}

__device__ __forceinline__ void report(const GemmParams& p, unsigned code) {
    if (p.status != nullptr) atomicCAS(p.status, 0u, code);
}

template <int KIND>
__device__ __forceinline__ void store_chunk(const GemmParams& p, uint32_t row, uint32_t col0, float (&acc)[32],
                                            uint32_t stage_row = 0, uint32_t unit0 = 0, bool c_staged = false) {
    // acc holds the fp32 accumulators of columns col0 .. col0+31 of `row` (clobbered).
    // stage_row == 0: write them to D (the caller guarantees row < M).
    // stage_row != 0: shared-memory address of this thread's 128-byte row of the warp's staging tile; the
    //   values go there (16-byte units unit0.., 128-byte swizzle) and a TMA store writes the tile later.  Rows
    //   at or beyond M are staged too (TMA drops them) but never read C.
    // c_staged: a TMA load has put this box of C into the staging tile (same units, same swizzle); C is read from
    //   there, unit by unit, right before the unit is overwritten with the result -- instead of 16-byte global
    //   loads that touch 32 different rows per warp instruction.
    const bool has_c = (p.C != nullptr) && (row < p.M);
    const uint32_t ncols = min(32u, p.N - col0);
    const uint32_t sw = (stage_row >> 7) & 7u;               // row index within the 8-row swizzle atom

    if constexpr (KIND == 0) {
        __half* drow = reinterpret_cast<__half*>(p.D) + size_t(row) * p.ldd + col0;
        const __half* crow = has_c ? reinterpret_cast<const __half*>(p.C) + size_t(row) * p.ldc + col0 : nullptr;
        const bool scale = has_c || p.alpha_re != 1.0f;
        if (scale) {
            if (has_c) {
                if (c_staged || (ncols == 32 && p.vec_c)) {
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const uint4 c4 = c_staged ? ld_shared_v4(stage_row + (((unit0 + q) ^ sw) << 4))
                                                  : __ldg(reinterpret_cast<const uint4*>(crow) + q);
                        const __half2* h = reinterpret_cast<const __half2*>(&c4);
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const float2 f = __half22float2(h[j]);
                            acc[q * 8 + 2 * j] = p.alpha_re * acc[q * 8 + 2 * j] + p.beta_re * f.x;
                            acc[q * 8 + 2 * j + 1] = p.alpha_re * acc[q * 8 + 2 * j + 1] + p.beta_re * f.y;
                        }
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (i < ncols) acc[i] = p.alpha_re * acc[i] + p.beta_re * __half2float(crow[i]);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[i] *= p.alpha_re;
            }
        }
        if (stage_row != 0) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint4 o;
                __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(acc[q * 8 + 2 * j], acc[q * 8 + 2 * j + 1]);
                st_shared_v4(stage_row + (((unit0 + q) ^ sw) << 4), o.x, o.y, o.z, o.w);
            }
        } else if (ncols == 32 && p.vec_d) {
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                uint4 o;
                __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
                for (int j = 0; j < 4; ++j) h[j] = __floats2half2_rn(acc[q * 8 + 2 * j], acc[q * 8 + 2 * j + 1]);
                reinterpret_cast<uint4*>(drow)[q] = o;
            }
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (i < ncols) drow[i] = __float2half_rn(acc[i]);
        }
    } else {
        float* drow = reinterpret_cast<float*>(p.D) + size_t(row) * p.ldd + col0;
        const float* crow = has_c ? reinterpret_cast<const float*>(p.C) + size_t(row) * p.ldc + col0 : nullptr;
        if (p.epi_mode == EPI_REAL) {
            if (has_c) {
                if (c_staged || (ncols == 32 && p.vec_c)) {
#pragma unroll
                    for (int q = 0; q < 8; ++q) {
                        float4 c4;
                        if (c_staged) {
                            const uint4 u = ld_shared_v4(stage_row + (((unit0 + q) ^ sw) << 4));
                            c4 = make_float4(__uint_as_float(u.x), __uint_as_float(u.y), __uint_as_float(u.z), __uint_as_float(u.w));
                        } else {
                            c4 = __ldg(reinterpret_cast<const float4*>(crow) + q);
                        }
                        acc[4 * q + 0] = p.alpha_re * acc[4 * q + 0] + p.beta_re * c4.x;
                        acc[4 * q + 1] = p.alpha_re * acc[4 * q + 1] + p.beta_re * c4.y;
                        acc[4 * q + 2] = p.alpha_re * acc[4 * q + 2] + p.beta_re * c4.z;
                        acc[4 * q + 3] = p.alpha_re * acc[4 * q + 3] + p.beta_re * c4.w;
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i)
                        if (i < ncols) acc[i] = p.alpha_re * acc[i] + p.beta_re * crow[i];
                }
            } else if (p.alpha_re != 1.0f) {
#pragma unroll
                for (int i = 0; i < 32; ++i) acc[i] *= p.alpha_re;
            }
        } else {
            // (re, im) pairs sit in adjacent columns; col0 and N are even here
            const bool scale = has_c || p.alpha_re != 1.0f || p.alpha_im != 0.0f;
            if (scale) {
#pragma unroll
                for (int q = 0; q < 8; ++q) {                // one 16-byte unit = two complex numbers
                    float cc[4] = {0.f, 0.f, 0.f, 0.f};
                    if (has_c) {
                        if (c_staged) {
                            const uint4 u = ld_shared_v4(stage_row + (((unit0 + q) ^ sw) << 4));
                            cc[0] = __uint_as_float(u.x); cc[1] = __uint_as_float(u.y);
                            cc[2] = __uint_as_float(u.z); cc[3] = __uint_as_float(u.w);
                        } else {
#pragma unroll
                            for (int e = 0; e < 4; e += 2)
                                if (uint32_t(4 * q + e) < ncols) {
                                    const float2 c2 = __ldg(reinterpret_cast<const float2*>(crow + 4 * q + e));
                                    cc[e] = c2.x; cc[e + 1] = c2.y;
                                }
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 4; e += 2) {
                        const int i = 4 * q + e;
                        const float re = acc[i], im = acc[i + 1];
                        acc[i] = p.alpha_re * re - p.alpha_im * im + p.beta_re * cc[e] - p.beta_im * cc[e + 1];
                        acc[i + 1] = p.alpha_re * im + p.alpha_im * re + p.beta_re * cc[e + 1] + p.beta_im * cc[e];
                    }
                }
            }
        }
        if (stage_row != 0) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
                st_shared_v4(stage_row + (((unit0 + q) ^ sw) << 4), __float_as_uint(acc[4 * q]),
                             __float_as_uint(acc[4 * q + 1]), __float_as_uint(acc[4 * q + 2]),
                             __float_as_uint(acc[4 * q + 3]));
        } else if (ncols == 32 && p.vec_d) {
#pragma unroll
            for (int q = 0; q < 8; ++q)
                reinterpret_cast<float4*>(drow)[q] =
                    make_float4(acc[4 * q], acc[4 * q + 1], acc[4 * q + 2], acc[4 * q + 3]);
        } else {
#pragma unroll
            for (int i = 0; i < 32; ++i)
                if (i < ncols) drow[i] = acc[i];
        }
    }
}

// Courier warp `courier` of `n_couriers` (all CTAs of the grid together): copies its share of the job list's
// batches, in list order, into the local replica and keeps the per-panel counts.  Every wait is bounded.
//
// Counting is batched: a courier adds what it has copied to the panel's counters when it moves on to another
// (panel, publishing or not) group of jobs, or runs out of work -- one fence per group instead of one per 8 KB.
// (A system-scope fence per batch limited the copy to ~130 GB/s.)  The publishing job of a panel comes first in
// the list, so a courier always hands in its published batches BEFORE it starts waiting on another GPU's flag.
__device__ __forceinline__ void fetch_flush(const FetchParams& f, const GemmParams& p, uint32_t lane, const FetchJob& J,
                                            uint32_t job, uint32_t job_batches, uint32_t count) {
    if (count == 0) return;
    const bool push = J.dst != nullptr;
    // the stores of every lane are performed before the counts below can be seen to include these batches:
    // readers of publish / notify flags are other GPUs (system scope), readers of ready_flags this GPU's loaders
    if (push || J.publish) __threadfence_system(); else __threadfence();
    __syncwarp();
    if (lane == 0) {
        if (push) {
            if (J.notify != nullptr && atomicAdd(f.job_done + job, count) + count == job_batches) {
                __threadfence_system();
                if (J.publish == FETCH_MULTICAST) multimem_red_max_release_sys(J.notify, f.epoch);
                else st_release_sys(J.notify, f.epoch);
                if (p.stats != nullptr) atomicMax(p.stats + 24 + min(J.panel, 7u), (unsigned long long)global_timer_ns());
            }
        } else {
            if (J.publish && atomicAdd(f.published + J.panel, count) + count == f.pub_need[J.panel]) {
                __threadfence_system();
                st_release_sys(f.pub_flags + J.panel, f.epoch);
                if (p.stats != nullptr) p.stats[24 + min(J.panel, 7u)] = global_timer_ns();
            }
            if (atomicAdd(f.arrived + J.panel, count) + count == f.need[J.panel]) {
                __threadfence();
                st_release_sys(f.ready_flags + J.panel, f.epoch);
                if (p.stats != nullptr) p.stats[J.panel] = global_timer_ns();
            }
        }
    }
    __syncwarp();
}

// One courier (a warp).  Batches are handed out by a global counter (f.next_batch), so every batch before the one a
// courier holds has been taken by somebody: the list is worked through in order whatever the couriers' speeds.
// `step` advances by at most one batch and never blocks for long when `may_block` is false -- that is what lets the
// epilogue warps, idle for most of a 256 x 512 tile, carry batches between two accumulator drains.
struct Courier {
    uint32_t job = 0, job_first = 0;             // current job and its first batch index
    uint32_t spr = 0, nseg = 0, nb = 0;
    FetchJob J;
    bool have = false, gate_open = false, done = false, holding = false;
    uint32_t cur = 0;                            // batch taken from the counter and not yet copied (if `holding`)
    uint32_t pend = 0;                           // batches of job PJ copied but not yet counted
    FetchJob PJ;
    uint32_t pend_job = 0, pend_nb = 0;
    uint64_t gate_t0 = 0;

    __device__ __forceinline__ void flush(const FetchParams& f, const GemmParams& p, uint32_t lane) {
        fetch_flush(f, p, lane, PJ, pend_job, pend_nb, pend);
        pend = 0;
    }

    __device__ __forceinline__ void step(const FetchParams& f, const GemmParams& p, uint32_t lane, bool may_block) {
        if (done) return;
        if (!holding) {
            uint32_t b = 0;
            if (lane == 0) b = atomicAdd(f.next_batch, 1u);
            b = __shfl_sync(0xffffffffu, b, 0);
            if (b >= f.total_batches) {
                flush(f, p, lane);
                done = true;
                return;
            }
            cur = b;
            holding = true;
            for (;;) {                           // the job that holds batch `cur` (batches only move forward)
                if (!have) {
                    if (job >= f.n_jobs) {       // inconsistent table: stop rather than read past it
                        flush(f, p, lane);
                        done = true;
                        return;
                    }
                    J = f.jobs[job];
                    spr = (J.bytes + 511u) / 512u;
                    nseg = J.rows * spr;
                    nb = fetch_job_batches(J.rows, J.bytes);
                    have = true;
                    gate_open = (J.gate == nullptr);
                    gate_t0 = 0;
                }
                if (cur < job_first + nb) break;
                job_first += nb;
                ++job;
                have = false;
            }
            if (pend != 0 && job != pend_job) flush(f, p, lane);   // hands a job's batches in BEFORE any wait on a flag
            PJ = J;
            pend_job = job;
            pend_nb = nb;
        }
        if (!gate_open) {
            // the piece is being produced elsewhere (another GPU's couriers or a copy engine): look at its flag
            uint32_t state = 0;                  // 0 closed, 1 open, 2 timed out
            if (lane == 0) {
                if (gate_t0 == 0) gate_t0 = global_timer_ns();
                for (;;) {
                    if (int(ld_acquire_sys(J.gate) - f.epoch) >= 0) { state = 1; break; }
                    if (global_timer_ns() - gate_t0 > p.wait_limit_ns) { state = 2; break; }
                    if (!may_block) break;
                    __nanosleep(256);
                }
            }
            state = __shfl_sync(0xffffffffu, state, 0);
            if (state == 2) {
                if (lane == 0) report(p, KS_TIMEOUT_FETCH);
                flush(f, p, lane);
                done = true;
                return;
            }
            if (state == 0) return;              // not yet: the caller has other things to look at
            (void)ld_acquire_sys(J.gate);        // every lane orders its own loads of the piece after the flag
            gate_open = true;
            if (p.stats != nullptr && J.rows == 0 && lane == 0) p.stats[24 + min(J.panel, 7u)] = global_timer_ns();
        }
        const uint32_t g0 = (cur - job_first) * FETCH_UNROLL;
        uint32_t row = g0 / (spr ? spr : 1u), cs = g0 - row * spr;
        uint4 v[FETCH_UNROLL];
        uint64_t off[FETCH_UNROLL];
#pragma unroll
        for (uint32_t u = 0; u < FETCH_UNROLL; ++u) {
            const uint32_t colb = cs * 512u + lane * 16u;
            const bool valid = (g0 + u < nseg) && (colb < J.bytes);
            off[u] = valid ? (uint64_t(J.row0 + row) * f.pitch + J.byte0 + colb) : ~0ull;
            if (valid) v[u] = ld_volatile_v4(J.src + off[u]);
            if (++cs == spr) { cs = 0; ++row; }
        }
        uint8_t* const dst = J.dst != nullptr ? J.dst : f.dst;
        if (J.dst != nullptr && J.publish == FETCH_MULTICAST) {
#pragma unroll
            for (uint32_t u = 0; u < FETCH_UNROLL; ++u)
                if (off[u] != ~0ull) multimem_st_v4(dst + off[u], v[u]);
        } else {
#pragma unroll
            for (uint32_t u = 0; u < FETCH_UNROLL; ++u)
                if (off[u] != ~0ull) *reinterpret_cast<uint4*>(dst + off[u]) = v[u];
        }
        ++pend;
        holding = false;
    }
};

// D forwarding: copies the part of this CTA's k-th tile that epilogue warp w (= warp 2 + w of the CTA: rows
// 32 * ((w + 2) & 3), the tensor-memory lanes that warp may read; accumulator w >> 2
// = tile columns [128a, +128) and [256 + 128a, +128)) staged in the CTA's ring to D, clipped at M and N.  One warp:
// lanes 0..15 carry the first 256-byte span of a row, lanes 16..31 the second.
__device__ __forceinline__ void forward_part(const FetchParams& f, const GemmParams& p, uint32_t lane, uint32_t w, uint32_t k,
                                             uint32_t worker, uint32_t n_workers, uint32_t cta_rank) {
    uint32_t tm, tn;
    tile_coords(worker + k * n_workers, p, tm, tn);
    const uint32_t q = (w + 2u) & 3u, a = w >> 2;
    const uint32_t row0 = (tm * 2 + cta_rank) * 128 + q * 32;
    const uint32_t colt = (lane < 16 ? 0u : 256u) + a * 128 + (lane & 15u) * 8;       // column within the tile
    const uint32_t col = tn * 512 + colt;
    const uint32_t rows = (row0 < p.M && col < p.N) ? min(32u, p.M - row0) : 0u;
    const uint8_t* src = f.fwd_stage + (uint64_t(blockIdx.x * 2 + (k & 1u)) * 128 + q * 32) * 1024 + colt * 2;
    uint8_t* dst = static_cast<uint8_t*>(p.D) + (uint64_t(row0) * p.ldd + col) * 2;
    const uint64_t dpitch = p.ldd * 2;
#pragma unroll 1
    for (uint32_t r0 = 0; r0 < rows; r0 += 4) {
        uint4 v[4];
#pragma unroll
        for (uint32_t u = 0; u < 4; ++u)
            if (r0 + u < rows) v[u] = ld_volatile_v4(src + uint64_t(r0 + u) * 1024);
#pragma unroll
        for (uint32_t u = 0; u < 4; ++u)
            if (r0 + u < rows) *reinterpret_cast<uint4*>(dst + uint64_t(r0 + u) * dpitch) = v[u];
    }
}

template <int KIND, int CTAS, int NACC, int FETCH, int BNV = 256>
__global__ void __launch_bounds__(GemmCfg<KIND, CTAS, NACC, FETCH, BNV>::THREADS, 1)
gemm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA0, const __grid_constant__ CUtensorMap tmA1,
                    const __grid_constant__ CUtensorMap tmB0, const __grid_constant__ CUtensorMap tmB1,
                    const __grid_constant__ CUtensorMap tmD, const __grid_constant__ CUtensorMap tmC, const GemmParams p,
                    const FetchParams f) {
    using Cfg = GemmCfg<KIND, CTAS, NACC, FETCH, BNV>;
    constexpr int STAGES = Cfg::STAGES;

    extern __shared__ uint8_t smem_raw[];
    // tiles need 1024-byte alignment for the 128-byte swizzle pattern
    const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t staging_base = smem_base + STAGES * Cfg::STAGE;   // 1024-byte aligned: 4 KB per epilogue warp
    const uint32_t bar_base = staging_base + Cfg::STAGING;
    const uint32_t full_bar = bar_base;                      // STAGES x 8 B
    const uint32_t empty_bar = bar_base + 8 * STAGES;        // STAGES x 8 B
    const uint32_t accf_bar = bar_base + 16 * STAGES;        // 2 x 8 B  accumulator full
    const uint32_t acce_bar = accf_bar + 16;                 // 2 x 8 B  accumulator empty
    const uint32_t tmem_slot = acce_bar + 16;                // 4 B
    const uint32_t cbar_base = acce_bar + 24;                // EPI_WARPS x 8 B: arrival of a box of C in a warp's staging tile
    volatile uint32_t* tmem_slot_ptr =
        reinterpret_cast<volatile uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
    // D forwarding mailbox: [w] parts published by epilogue warp w, [8 + w] parts of that warp copied to D
    volatile uint32_t* mbox = reinterpret_cast<volatile uint32_t*>(smem_raw + (bar_base + 256 - smem_u32(smem_raw)));
    bool fwd = false;
    if constexpr (FETCH > 0 && NACC == 2) fwd = f.fwd_stage != nullptr;

    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31;
    const uint32_t cta_rank = (CTAS == 2) ? cluster_ctarank() : 0u;
    const bool leader = (cta_rank == 0);
    const uint32_t n_workers = gridDim.x / CTAS;             // CTAs (or pairs) walking the tile list
    const uint32_t worker = blockIdx.x / CTAS;
    const uint32_t n_tiles = p.tiles_m * p.tiles_n;
    const uint32_t n_kb = (p.K + Cfg::BK - 1) / Cfg::BK;
    const uint64_t limit = p.wait_limit_ns;
    // k-blocks per TMEM accumulation chain: a few when the epilogue sums chunks in registers, else all
    const uint32_t chunk_kb = Cfg::PROMOTE ? uint32_t(Cfg::CHUNK_KB) : n_kb;
    const uint32_t n_chunks = (n_kb + chunk_kb - 1) / chunk_kb;

    if constexpr (FETCH > 0) {
        if (threadIdx.x >= 32 && threadIdx.x < 48) mbox[threadIdx.x - 32] = 0u;
    }
    if (threadIdx.x == 0) {
        if (p.stats != nullptr && blockIdx.x == 0) p.stats[16] = global_timer_ns();
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(full_bar + 8 * s, 1);
            mbar_init(empty_bar + 8 * s, 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(accf_bar + 8 * a, 1);
            mbar_init(acce_bar + 8 * a, Cfg::ACC_ARRIVALS);
        }
        for (int w = 0; w < Cfg::EPI_WARPS; ++w) mbar_init(cbar_base + 8 * w, 1);
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc<CTAS>(tmem_slot, Cfg::TMEM_COLS);
        tmem_relinquish<CTAS>();
    }
    tc_fence_before_sync();
    if constexpr (CTAS == 2) cluster_sync_all(); else __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot_ptr;
    // 3xTF32: the pass that wrote the operand planes may still be running (programmatic dependent launch)
    if constexpr (KIND == 1) griddep_wait();

    if (warp == 0) {
        // ------------------------------------------------------------------ TMA producer
        if (lane == 0) {
            tma_prefetch_desc(&tmA0);
            tma_prefetch_desc(&tmB0);
            if constexpr (KIND == 1) { tma_prefetch_desc(&tmA1); tma_prefetch_desc(&tmB1); }
            const uint32_t full_target = (CTAS == 2) ? map_to_cta(full_bar, 0) : full_bar;
            uint32_t s = 0, ph = 0, my_iter = 0, cur_panel = 0xFFFFFFFFu;
            bool ok = true;
            for (uint32_t t = worker; t < n_tiles && ok; t += n_workers, ++my_iter) {
                if (p.sync_on && leader && my_iter > 0) {
                    atomicAdd(&g_wave_ticket, 1u);           // this worker has issued all loads of its previous tile
                    const uint32_t done_before = min(n_tiles, my_iter * n_workers);   // tiles of earlier rounds
                    const unsigned target = p.sync_base + done_before;
                    const uint64_t t0 = global_timer_ns();
                    while (int(*reinterpret_cast<volatile unsigned*>(&g_wave_ticket) - target) < 0) {
                        if (global_timer_ns() - t0 > p.sync_limit_ns) break;      // soft: go on alone
                    }
                }
                uint32_t tm, tn;
                const uint32_t panel = tile_coords(t, p, tm, tn);
                if (p.panel_flags != nullptr && panel != cur_panel) {
                    // B's panel may still be on its way: wait for its arrival flag, then make the data it
                    // guards visible to the TMA loads
                    const uint64_t t0 = global_timer_ns();
                    bool arrived = true, waited = false;
                    while (int(ld_acquire_sys(p.panel_flags + panel) - p.panel_epoch) < 0) {
                        waited = true;
                        if (global_timer_ns() - t0 > limit) { arrived = false; break; }
                    }
                    if (waited && p.stats != nullptr) {
                        atomicAdd(p.stats + 18, (unsigned long long)(global_timer_ns() - t0));
                        atomicAdd(p.stats + 19, 1ull);
                    }
                    if (!arrived) {
                        report(p, KS_TIMEOUT_PANEL);
                        ok = false;
                        break;
                    }
                    fence_proxy_async_all();
                    cur_panel = panel;
                }
                const int32_t row0 = int32_t((tm * CTAS + cta_rank) * Cfg::BM);
                const int32_t col0 = int32_t(tn * Cfg::BN_TILE + cta_rank * Cfg::BN_LOAD);
                int32_t conv_x0 = 0, conv_y0 = 0;
                if constexpr (KIND == 1) {
                    if (p.conv_tw != 0) {            // every CTA of a pair has an M tile of its own
                        const uint32_t tmi = tm * CTAS + cta_rank;
                        conv_x0 = int32_t((tmi % p.conv_tiles_x) * p.conv_tw);
                        conv_y0 = int32_t((tmi / p.conv_tiles_x) * (uint32_t(Cfg::BM) / p.conv_tw));
                    }
                }
                for (uint32_t kb = 0; kb < n_kb; ++kb) {
                    if (!mbar_wait_bounded(empty_bar + 8 * s, ph ^ 1u, limit)) {
                        report(p, KS_TIMEOUT_PRODUCER);
                        ok = false;
                        break;
                    }
                    const uint32_t stage = smem_base + s * Cfg::STAGE;
                    const uint32_t fb = full_target + 8 * s;
                    if (leader) mbar_arrive_expect_tx(full_bar + 8 * s, uint32_t(Cfg::STAGE) * CTAS);
                    const int32_t k0 = int32_t(kb * Cfg::BK);
#pragma unroll
                    for (int pl = 0; pl < Cfg::NPL; ++pl) {
                        const CUtensorMap* ma = (pl == 0) ? &tmA0 : &tmA1;
                        const CUtensorMap* mb = (pl == 0) ? &tmB0 : &tmB1;
                        const uint32_t a_dst = stage + pl * Cfg::A_TILE;
                        const uint32_t b_dst = stage + Cfg::NPL * Cfg::A_TILE + pl * Cfg::B_TILE;
                        if constexpr (CTAS == 2 && KIND == 1) {
                            if (p.conv_tw != 0)
                                tma_load_4d_pair(a_dst, ma, fb, int32_t((kb % p.conv_kbi) * Cfg::BK), conv_x0,
                                                 int32_t(kb / p.conv_kbi), conv_y0);
                            else
                                tma_load_2d_pair(a_dst, ma, fb, k0, row0);
                        } else if constexpr (CTAS == 2) {
                            tma_load_2d_pair(a_dst, ma, fb, k0, row0);
                        } else if constexpr (KIND == 1) {
                            if (p.conv_tw != 0)
                                tma_load_4d(a_dst, ma, fb, int32_t((kb % p.conv_kbi) * Cfg::BK), conv_x0,
                                            int32_t(kb / p.conv_kbi), conv_y0);
                            else
                                tma_load_2d(a_dst, ma, fb, k0, row0);
                        } else {
                            tma_load_2d(a_dst, ma, fb, k0, row0);
                        }
                        if (p.b_chunked_map) {
                            // all B_CHUNKS chunks of this stage in one instruction: the issuing thread, not
                            // the memory system, limits how fast stages can be refilled
                            if constexpr (CTAS == 2) tma_load_3d_pair(b_dst, mb, fb, 0, k0, col0 / Cfg::CHUNK_N);
                            else tma_load_3d(b_dst, mb, fb, 0, k0, col0 / Cfg::CHUNK_N);
                        } else {
#pragma unroll
                            for (int j = 0; j < Cfg::B_CHUNKS; ++j) {
                                if constexpr (CTAS == 2)
                                    tma_load_2d_pair(b_dst + j * Cfg::B_CHUNK_BYTES, mb, fb, col0 + j * Cfg::CHUNK_N, k0);
                                else
                                    tma_load_2d(b_dst + j * Cfg::B_CHUNK_BYTES, mb, fb, col0 + j * Cfg::CHUNK_N, k0);
                            }
                        }
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
            if (p.sync_on && leader && my_iter > 0) atomicAdd(&g_wave_ticket, 1u);   // ticket of the last tile
            // tail: every stage this CTA filled has been released by the MMA side, so no
            // arrival (possibly from the peer CTA) can land after this CTA has exited
            if (ok) {
                for (int i = 0; i < STAGES; ++i) {
                    if (!mbar_wait_bounded(empty_bar + 8 * s, ph ^ 1u, limit)) {
                        report(p, KS_TIMEOUT_TAIL);
                        break;
                    }
                    if (++s == STAGES) { s = 0; ph ^= 1u; }
                }
            }
        }
    } else if (warp == 1) {
        // ------------------------------------------------------------------ MMA issuer
        if (leader && lane == 0) {
            // A, K-major: rows of 128 B, 8-row swizzle atoms 1024 B apart.
            constexpr uint64_t DESC_A = smem_desc(SMEM_LAYOUT_SW128, 16, 1024);
            // B, MN-major: 128-byte chunks of N, B_CHUNK_BYTES apart; k rows 128 B apart, grouped by
            // swizzle atom (8 rows = 1024 B for 16-bit operands, 4 rows = 512 B for 32-bit operands).
            constexpr uint64_t DESC_B = (KIND == 0) ? smem_desc(SMEM_LAYOUT_SW128, Cfg::B_CHUNK_BYTES, 1024)
                                                    : smem_desc(SMEM_LAYOUT_SW128_BASE32B, Cfg::B_CHUNK_BYTES, 512);
            constexpr uint32_t A_KSTEP = 32;                                          // UMMA_K elements along a 128 B row
            constexpr uint32_t B_KSTEP = Cfg::UMMA_K * 128;                           // UMMA_K rows of 128 B
            const uint32_t peer_empty = (CTAS == 2) ? map_to_cta(empty_bar, 1) : 0u;
            const uint32_t peer_accf = (CTAS == 2) ? map_to_cta(accf_bar, 1) : 0u;
            uint32_t s = 0, ph = 0, it = 0;          // `it` counts accumulation chains (chunks)
            bool ok = true;
            const bool timed = p.stats != nullptr;
            uint64_t w_full = 0, w_acc = 0;
            const uint64_t t_loop = timed ? global_timer_ns() : 0;

            for (uint32_t t = worker; t < n_tiles && ok; t += n_workers) {
                for (uint32_t c = 0; c < n_chunks && ok; ++c, ++it) {
                    // NACC 1: chains alternate between the two TMEM accumulators; NACC 2: a tile owns both
                    const uint32_t a = (NACC == 2) ? 0u : (it & 1u);
                    const uint32_t aph = (NACC == 2) ? (it & 1u) : ((it >> 1) & 1u);
                    const uint64_t ta = timed ? global_timer_ns() : 0;
                    bool freed = mbar_wait_bounded(acce_bar + 8 * a, aph ^ 1u, limit);
                    if (NACC == 2 && freed) freed = mbar_wait_bounded(acce_bar + 8, aph ^ 1u, limit);
                    if (timed) w_acc += global_timer_ns() - ta;
                    if (!freed) {
                        report(p, KS_TIMEOUT_MMA_ACC);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t d_tmem = tmem_base + a * Cfg::BN;
                    const uint32_t kb_end = min(n_kb, (c + 1) * chunk_kb);
                    for (uint32_t kb = c * chunk_kb; kb < kb_end; ++kb) {
                        const uint64_t tf = timed ? global_timer_ns() : 0;
                        const bool filled = mbar_wait_bounded(full_bar + 8 * s, ph, limit);
                        if (timed) w_full += global_timer_ns() - tf;
                        if (!filled) {
                            report(p, KS_TIMEOUT_MMA_FULL);
                            ok = false;
                            break;
                        }
                        tc_fence_after_sync();
                        const uint32_t stage = smem_base + s * Cfg::STAGE;
                        const uint32_t a0 = stage, b0 = stage + Cfg::NPL * Cfg::A_TILE;
#pragma unroll
                        for (int k = 0; k < Cfg::BK / Cfg::UMMA_K; ++k) {
                            const uint32_t acc_flag = ((kb - c * chunk_kb) | uint32_t(k)) ? 1u : 0u;
                            if constexpr (KIND == 0) {
                                const uint64_t da = smem_desc_at(DESC_A, a0 + k * A_KSTEP);
#pragma unroll
                                for (int h = 0; h < NACC; ++h)      // accumulator h: this CTA's chunks [2h, 2h+2) when NACC = 2
                                    umma_ss<0, CTAS>(d_tmem + h * Cfg::BN, da,
                                                     smem_desc_at(DESC_B, b0 + h * (Cfg::B_TILE / NACC) + k * B_KSTEP),
                                                     Cfg::IDESC, acc_flag);
                            } else {
                                const uint64_t a_hi = smem_desc_at(DESC_A, a0 + k * A_KSTEP);
                                const uint64_t a_lo = smem_desc_at(DESC_A, a0 + Cfg::A_TILE + k * A_KSTEP);
                                const uint64_t b_hi = smem_desc_at(DESC_B, b0 + k * B_KSTEP);
                                const uint64_t b_lo = smem_desc_at(DESC_B, b0 + Cfg::B_TILE + k * B_KSTEP);
                                // small terms first, the dominant hi*hi product last
                                umma_ss<1, CTAS>(d_tmem, a_lo, b_hi, Cfg::IDESC, acc_flag);
                                umma_ss<1, CTAS>(d_tmem, a_hi, b_lo, Cfg::IDESC, 1u);
                                umma_ss<1, CTAS>(d_tmem, a_hi, b_hi, Cfg::IDESC, 1u);
                            }
                        }
                        umma_commit<CTAS>(empty_bar + 8 * s);             // stage free once these MMAs retire
                        if constexpr (CTAS == 2) umma_commit<CTAS>(peer_empty + 8 * s);
                        if (++s == STAGES) { s = 0; ph ^= 1u; }
                    }
                    if (ok) {
#pragma unroll
                        for (int h = 0; h < NACC; ++h) {
                            umma_commit<CTAS>(accf_bar + 8 * (a + h));    // chain complete
                            if constexpr (CTAS == 2) umma_commit<CTAS>(peer_accf + 8 * (a + h));
                        }
                    }
                }
            }
            if (timed) {
                atomicAdd(p.stats + 20, (unsigned long long)w_full);
                atomicAdd(p.stats + 21, (unsigned long long)w_acc);
                atomicAdd(p.stats + 22, (unsigned long long)(global_timer_ns() - t_loop));
                atomicAdd(p.stats + 23, 1ull);
            }
            // tail: both accumulators drained by every epilogue warp (of both CTAs)
            if (ok) {
                for (int i = 0; i < 2; ++i) {
                    const uint32_t a = (NACC == 2) ? uint32_t(i) : (it & 1u);
                    const uint32_t aph = (NACC == 2) ? (it & 1u) : ((it >> 1) & 1u);
                    if (NACC == 1) ++it;
                    if (!mbar_wait_bounded(acce_bar + 8 * a, aph ^ 1u, limit)) {
                        report(p, KS_TIMEOUT_TAIL);
                        break;
                    }
                }
            }
        }
    } else if (FETCH > 0 && warp >= 2u + Cfg::EPI_WARPS) {
        // ------------------------------------------------------------------ couriers (B from the other GPUs)
        Courier c;
        if (!fwd) {
            while (!c.done) c.step(f, p, lane, true);
        } else {
            // two couriers per CTA: each also forwards the finished parts of four epilogue warps to D, between
            // batches of B (a part is 32 KB once per tile: B is hardly delayed, and the ring gives D a tile's time)
            const uint32_t cw = warp - (2u + Cfg::EPI_WARPS);
            const uint32_t my_tiles = n_tiles > worker ? (n_tiles - worker - 1) / n_workers + 1 : 0u;
            uint32_t sent[4] = {0u, 0u, 0u, 0u};
            uint64_t idle_since = global_timer_ns();
            for (;;) {
                bool progressed = false, all_sent = true;
#pragma unroll
                for (uint32_t j = 0; j < 4; ++j) {
                    const uint32_t w = cw + 2 * j;
                    if (sent[j] < my_tiles) {
                        uint32_t seq = 0;
                        if (lane == 0) seq = mbox[w];
                        seq = __shfl_sync(0xffffffffu, seq, 0);
                        if (seq > sent[j]) {
                            __threadfence();                 // the part's bytes, written before the count
                            forward_part(f, p, lane, w, sent[j], worker, n_workers, cta_rank);
                            ++sent[j];
                            __syncwarp();
                            if (lane == 0) mbox[8 + w] = sent[j];     // the ring slot may be overwritten
                            progressed = true;
                        }
                        if (sent[j] < my_tiles) all_sent = false;
                    }
                }
                if (!c.done) {
                    c.step(f, p, lane, false);               // its own waits are bounded
                    idle_since = global_timer_ns();
                    continue;
                }
                if (all_sent) break;
                if (progressed) {
                    idle_since = global_timer_ns();
                } else {
                    if (global_timer_ns() - idle_since > limit) {       // the epilogue gave up: nothing more will come
                        if (lane == 0) report(p, KS_TIMEOUT_FETCH);
                        break;
                    }
                    __nanosleep(200);
                }
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 2..)
        const uint32_t quarter = warp & 3u;                  // TMEM lanes [32*quarter, +32) belong to this warp
        const uint32_t colpart = (warp - 2u) >> 2;           // which EPI_COLS-wide slice of the 256 columns
        const uint32_t acce_target = (CTAS == 2) ? map_to_cta(acce_bar, 0) : acce_bar;
        const uint32_t stage_warp = staging_base + (warp - 2u) * 4096u;   // this warp's 32 x 128-byte staging tile
        const uint32_t stage_row = p.d_tma ? stage_warp + lane * 128u : 0u;
        constexpr uint32_t BOX_COLS = 128 / ((KIND == 0) ? 2 : 4);        // output columns per 128-byte row
        if (p.d_tma && lane == 0) tma_prefetch_desc(&tmD);
        if (p.c_tma && lane == 0) tma_prefetch_desc(&tmC);
        const uint32_t cbar = cbar_base + 8 * (warp - 2u);
        uint32_t cph = 0;                                    // phase of cbar
        // Brings the box of C at (box_col, box_row) into this warp's staging tile; every lane returns once the
        // data is there.  The previous TMA store must already have finished reading the tile.
        auto fetch_c_box = [&](uint32_t box_col, uint32_t box_row) -> bool {
            if (lane == 0) {
                mbar_arrive_expect_tx(cbar, 4096u);
                tma_load_2d(stage_warp, &tmC, cbar, int32_t(box_col), int32_t(box_row));
            }
            const bool got = mbar_wait_bounded(cbar, cph, limit);
            cph ^= 1u;
            return got;
        };
        // TMA drops rows at or beyond M exactly, but it was seen to clip the column edge in 16-byte units, so a box
        // that crosses an edge N which is not 16-byte aligned is written by predicated per-thread stores instead
        const bool ragged_n = ((p.N * ((KIND == 0) ? 2u : 4u)) & 15u) != 0u;
        uint32_t it = 0;                                     // accumulation chains seen so far
        bool ok = true;
        Courier courier;                                     // used when FETCH > 0: see the wait below
        for (uint32_t t = worker; t < n_tiles && ok; t += n_workers) {
            uint32_t tm, tn;
            tile_coords(t, p, tm, tn);
            const uint32_t row = (tm * CTAS + cta_rank) * Cfg::BM + quarter * 32 + lane;
            const uint32_t colbase = tn * Cfg::BN + colpart * Cfg::EPI_COLS;
            if constexpr (Cfg::PROMOTE) {
                float sum[Cfg::EPI_COLS];
#pragma unroll
                for (int i = 0; i < Cfg::EPI_COLS; ++i) sum[i] = 0.f;
                for (uint32_t c = 0; c < n_chunks && ok; ++c, ++it) {
                    const uint32_t a = it & 1u, aph = (it >> 1) & 1u;
                    if (!mbar_wait_bounded(accf_bar + 8 * a, aph, limit)) {
                        if (lane == 0) report(p, KS_TIMEOUT_EPILOGUE);
                        ok = false;
                        break;
                    }
                    tc_fence_after_sync();
                    const uint32_t taddr = tmem_base + a * Cfg::BN + colpart * Cfg::EPI_COLS + ((quarter * 32u) << 16);
#pragma unroll
                    for (int q = 0; q < Cfg::EPI_COLS / 32; ++q) {
                        if (colbase + q * 32 < p.N) {        // uniform across the warp
                            uint32_t v[32];
                            tmem_ld_32x32(taddr + q * 32, v);
                            tmem_ld_wait();
#pragma unroll
                            for (int i = 0; i < 32; ++i) sum[q * 32 + i] += __uint_as_float(v[i]);
                        }
                    }
                    tc_fence_before_sync();
                    __syncwarp();
                    if (lane == 0) {
                        if constexpr (CTAS == 2) mbar_arrive_cluster(acce_target + 8 * a);
                        else mbar_arrive(acce_bar + 8 * a);
                    }
                }
                if (ok && (p.d_tma || row < p.M)) {
                    const uint32_t warp_row0 = (tm * CTAS + cta_rank) * Cfg::BM + quarter * 32;
#pragma unroll
                    for (int q = 0; q < Cfg::EPI_COLS / 32; ++q) {
                        const uint32_t col0 = colbase + q * 32;
                        if (col0 < p.N) {                    // uniform across the warp
                            float part[32];
#pragma unroll
                            for (int i = 0; i < 32; ++i) part[i] = sum[q * 32 + i];
                            if (p.d_tma && !(ragged_n && col0 + BOX_COLS > p.N)) {
                                if (lane == 0) bulk_wait_read_all();     // the previous box has left the staging tile
                                __syncwarp();
                                const bool c_box = p.c_tma && warp_row0 < p.M;
                                if (c_box && !fetch_c_box(col0, warp_row0)) {
                                    if (lane == 0) report(p, KS_TIMEOUT_EPILOGUE);
                                    ok = false;
                                    break;
                                }
                                store_chunk<KIND>(p, row, col0, part, stage_row, 0, c_box);
                                fence_proxy_async_smem();
                                __syncwarp();
                                if (lane == 0 && warp_row0 < p.M) {
                                    if (p.conv_tw != 0) {   // this warp's 32 rows: 32 consecutive x of one output row
                                        const uint32_t r0 = quarter * 32, tmi = tm * CTAS + cta_rank;
                                        tma_store_3d(&tmD, stage_warp, int32_t(col0),
                                                     int32_t((tmi % p.conv_tiles_x) * p.conv_tw + r0 % p.conv_tw),
                                                     int32_t((tmi / p.conv_tiles_x) * (uint32_t(Cfg::BM) / p.conv_tw) + r0 / p.conv_tw));
                                    } else {
                                        tma_store_2d(&tmD, stage_warp, int32_t(col0), int32_t(warp_row0));
                                    }
                                    bulk_commit_group();
                                }
                            } else if (row < p.M) {
                                store_chunk<KIND>(p, row, col0, part);
                            }
                        }
                    }
                }
            } else {
                // NACC 1: tiles alternate between the accumulators; NACC 2: warps 2..5 drain accumulator 0,
                // warps 6..9 accumulator 1 of every tile
                const uint32_t a = (NACC == 2) ? colpart : (it & 1u);
                const uint32_t aph = (NACC == 2) ? (it & 1u) : ((it >> 1) & 1u);
                if constexpr (FETCH > 0) {
                    // this warp has nothing to do until the tile's MMAs are done: carry batches of B meanwhile
                    while (!courier.done && !mbar_try_wait(accf_bar + 8 * a, aph)) courier.step(f, p, lane, false);
                    courier.flush(f, p, lane);           // nothing copied stays uncounted while the tile is drained
                }
                if (!mbar_wait_bounded(accf_bar + 8 * a, aph, limit)) {
                    if (lane == 0) report(p, KS_TIMEOUT_EPILOGUE);
                    ok = false;
                    break;
                }
                tc_fence_after_sync();
                const uint32_t taddr = tmem_base + a * Cfg::BN + ((quarter * 32u) << 16);
                if (fwd && it >= 2) {
                    // D forwarding: this part goes into ring slot it & 1; the part staged there two tiles ago must
                    // have been copied to D (it had a whole tile's time: normally no wait at all)
                    uint32_t gone = 1;
                    if (lane == 0) {
                        const uint64_t t0 = global_timer_ns();
                        while (mbox[8 + (warp - 2u)] + 2u <= it) {
                            if (global_timer_ns() - t0 > limit) { gone = 0; break; }
                            __nanosleep(100);
                        }
                    }
                    gone = __shfl_sync(0xffffffffu, gone, 0);
                    if (!gone) {
                        if (lane == 0) report(p, KS_TIMEOUT_EPILOGUE);
                        ok = false;
                        break;
                    }
                }
#pragma unroll 1
                for (uint32_t c = 0; c < Cfg::EPI_COLS / 32; ++c) {
                    // accumulator column 32c -> matrix column.  NACC 2: columns 0..127 of accumulator h come from
                    // CTA 0's B columns [128h, +128) of the tile, columns 128..255 from CTA 1's (256 further on)
                    const uint32_t col0 = (NACC == 2) ? tn * Cfg::BN_TILE + ((c * 32) >> 7) * 256 + a * 128 + ((c * 32) & 127)
                                                      : colbase + c * 32;
                    if (col0 >= p.N) break;                  // uniform across the warp
                    uint32_t v[32];
                    tmem_ld_32x32(taddr + c * 32, v);
                    tmem_ld_wait();
                    float acc[32];
#pragma unroll
                    for (int i = 0; i < 32; ++i) acc[i] = __uint_as_float(v[i]);
                    const uint32_t box_col0 = col0 - (c & (BOX_COLS / 32 - 1)) * 32;
                    if (p.d_tma && !(ragged_n && box_col0 + BOX_COLS > p.N)) {
                        // two 32-column chunks fill one 64-column (128-byte) box of fp16 output
                        const uint32_t half = c & (BOX_COLS / 32 - 1);
                        const uint32_t warp_row0_c = (tm * CTAS + cta_rank) * Cfg::BM + quarter * 32;
                        const bool c_box = p.c_tma && warp_row0_c < p.M;
                        if (half == 0) {
                            if (lane == 0) bulk_wait_read_all();         // the previous box has left the staging tile
                            __syncwarp();
                            if (c_box && !fetch_c_box(box_col0, warp_row0_c)) {
                                if (lane == 0) report(p, KS_TIMEOUT_EPILOGUE);
                                ok = false;
                                break;
                            }
                        }
                        store_chunk<KIND>(p, row, col0, acc, stage_row, half * 4, c_box);
                        if (half == BOX_COLS / 32 - 1 || col0 + 32 >= p.N) {
                            const uint32_t warp_row0 = (tm * CTAS + cta_rank) * Cfg::BM + quarter * 32;
                            fence_proxy_async_smem();
                            __syncwarp();
                            if (fwd) {
                                // into this CTA's ring in local memory (tmC maps it: 512 columns, 128 rows per slot)
                                if (lane == 0) {
                                    tma_store_2d(&tmC, stage_warp, int32_t(col0 - half * 32 - tn * Cfg::BN_TILE),
                                                 int32_t((blockIdx.x * 2 + (it & 1u)) * Cfg::BM + quarter * 32));
                                    bulk_commit_group();
                                }
                            } else if (lane == 0 && warp_row0 < p.M) {
                                tma_store_2d(&tmD, stage_warp, int32_t(col0 - half * 32), int32_t(warp_row0));
                                bulk_commit_group();
                            }
                        }
                    } else if (row < p.M) {
                        store_chunk<KIND>(p, row, col0, acc);
                    }
                }
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) {
                    if constexpr (CTAS == 2) mbar_arrive_cluster(acce_target + 8 * a);
                    else mbar_arrive(acce_bar + 8 * a);
                }
                if (fwd) {
                    // the part is complete in the ring: hand it to this CTA's couriers
                    if (lane == 0) {
                        bulk_wait_all();
                        fence_proxy_async_all();
                        __threadfence();
                        mbox[warp - 2u] = it + 1u;
                    }
                    __syncwarp();
                }
                ++it;
            }
        }
        if constexpr (FETCH > 0) {
            // no tiles left (or none at all) for this worker: full-time courier until the list is done
            while (!courier.done) courier.step(f, p, lane, true);
        }
    }

    if (warp >= 2 && warp < 2u + Cfg::EPI_WARPS && lane == 0 && p.d_tma) bulk_wait_all();   // this thread's output boxes are in memory

    // ---------------------------------------------------------------------- teardown
    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc<CTAS>(tmem_base, Cfg::TMEM_COLS);
    }
    if constexpr (CTAS == 2) cluster_sync_all();
    if (threadIdx.x == 0 && p.stats != nullptr) atomicMax(p.stats + 17, (unsigned long long)global_timer_ns());
}

}  // namespace dxb
