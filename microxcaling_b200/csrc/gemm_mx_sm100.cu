// Block-scaled MX GEMM for sm_100a:  C[b] = A[b] (M x K) * B[b]^T (N x K)
//
// Operands are the packed outputs of the MX quantizer: one fp8-container code
// per element (K contiguous) and one E8M0 scale per 32 elements, the scales in
// the 512-byte chunk layout tensor memory wants (see mxq_sf_offset in mxq.h).
// The products are formed by tcgen05.mma kind::mxf8f6f4 with the block scales
// applied by the tensor core, accumulated in fp32 in tensor memory -- this
// replaces the reference's "dequantize, then fp32 / bf16 library GEMM"
// (mx/linear.py:83-86, mx/matmul.py:83-86, mx/bmm.py:56-59).  The epilogue
// applies the bfloat rounding of mx_specs (and the bias add with its second
// rounding, mx/linear.py:88-96) while the accumulator is read out.
//
// One persistent CTA per SM, 320 threads:
//   warp 0      TMA producer: A and B tiles (128-byte swizzle) and the scale
//               chunks into a STAGES-deep shared-memory ring
//   warp 1      MMA issuer: copies the scales to tensor memory (tcgen05.cp),
//               issues four K=32 MMAs per 128-wide K block, commits the stage
//               back to the producer and finished accumulators to the epilogue
//   warps 2..9  epilogue: two warps per 32-lane quarter of tensor memory read
//               half of the accumulator columns each (tcgen05.ld), round, and
//               store through a swizzled staging tile with TMA
// Accumulators are double buffered in tensor memory so the epilogue of one
// tile overlaps the main loop of the next; a second kernel runs CTA pairs
// (cta_group::2) on 256 x 256 tiles.  All waits are bounded; on time-out the
// kernel records a status word, drains and exits.
#include <cuda.h>
#include <algorithm>
#include <cstring>
#include <mutex>
#include "mxq_common.cuh"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

namespace mxq {

// Operand stages of the CTA-pair kernel (5 leaves room for 128-byte-wide output boxes).
#ifndef MXQ_PAIR_STAGES
#define MXQ_PAIR_STAGES 5
#endif
#ifndef MXQ_PAIR_BOX
#define MXQ_PAIR_BOX 128
#endif

constexpr int kBM = 128;          // tile rows (MMA M per CTA)
constexpr int kBK = 128;          // K bytes per stage = four MMA K steps
constexpr int kEpiWarps = 8;       // two per tensor-memory lane quarter
constexpr int kGemmThreads = 64 + 32 * kEpiWarps;
constexpr int kSfChunk = 512;     // bytes of scales per 128 rows x 128 K

// fp32 accumulator -> bfloat grid: integer rounding on the raw bits (formats
// with eight exponent bits share fp32's exponent layout), branch-free.  The
// constants are derived once per launch from (mode, bits dropped).
struct OutRound {
    uint32_t add;       // half step (half-away), half step minus one (half-even), 0 (toward zero / off)
    uint32_t even_on;   // 1 for half-even
    uint32_t keep;      // mask of the bits kept
    uint32_t drop;
};
__device__ __forceinline__ uint32_t round_out_bits(uint32_t u, const OutRound& k) {
    const uint32_t mag = u & 0x7fffffffu;
    uint32_t r = (mag + k.add + ((mag >> k.drop) & k.even_on)) & k.keep;
    r = mag >= kInf ? mag : r;                    // Inf / NaN pass through
    return r | (u & 0x80000000u);
}

struct GemmArgs {
    const uint8_t* sfa;
    const uint8_t* sfb;
    void* c;
    const void* bias;           // fp32 [N] or null
    int* status;                // device status word
    int64_t M, N, K, batch;
    int64_t m_tiles, n_tiles, k_blocks;
    int64_t sfa_rows128, sfb_rows128;   // 128-row chunks per batch element
    uint32_t idesc;
    int out_dtype;              // DT_F32 or DT_BF16
    OutRound rnd;               // bfloat rounding of the result
    int epi_kind;               // 0/1/2: bf16 out, bfloat16 rounding nearest/floor/even, no bias; 3: generic
    int c_tma;                  // output written by TMA stores (row pitch multiple of 16 bytes)
    int group_m;                // tile-rows per raster group
    int64_t rows_per_dest;      // > 0: output rows [d * rows_per_dest, (d+1) * rows_per_dest) go to destination d
};

// Output tensor maps.  A plain GEMM uses m[0].  The scattering GEMM of a
// row-parallel layer has one map per destination buffer (its own memory or a
// peer GPU's, mapped into this process): every 128-row tile of the result is
// stored straight into the buffer of the rank that owns those rows, tile by
// tile while the other tiles are still being computed.
constexpr int kMaxDests = 8;
struct OutMaps {
    CUtensorMap m[kMaxDests];
};

// Shared memory of the single-CTA kernel.  The epilogue staging ring holds, per
// epilogue warp, NBUF boxes of 32 rows x BOX bytes (BOX = 64 or 128, swizzled
// like the output tensor map).
template <int BN, int STAGES, int BOX, int NBUF>
struct GemmSmem {
    static constexpr int kA = kBM * kBK;
    static constexpr int kB = BN * kBK;
    static constexpr int kSFA = kSfChunk;
    static constexpr int kSFB = (BN / 128) * kSfChunk;
    static constexpr int kStage = kA + kB + kSFA + kSFB;
    static constexpr int kStgOff = (STAGES * kStage + 1023) / 1024 * 1024;
    static constexpr int kStgWarp = 32 * BOX * NBUF;
    static constexpr int kBarOff = kStgOff + kEpiWarps * kStgWarp;
    static constexpr int kTotal = kBarOff + 256 + 1024;   // barriers + alignment slack
};

// Tile order: within a batch element, groups of kGroupM tile-rows are walked
// column by column (m fastest inside a group), so the CTAs running at the same
// time share a few A row-panels and a few B column-panels in L2 instead of
// streaming the whole of B once per tile row.
constexpr int kGroupM = 16;
__device__ __forceinline__ void tile_coords(int64_t t, const GemmArgs& g, int64_t tiles_per_batch,
                                            int64_t& bi, int64_t& mt, int64_t& nt) {
    bi = t / tiles_per_batch;
    const int64_t r = t % tiles_per_batch;
    const int64_t per_group = (int64_t)g.group_m * g.n_tiles;
    const int64_t grp = r / per_group;
    const int64_t i = r % per_group;
    const int64_t rows = min((int64_t)g.group_m, g.m_tiles - grp * g.group_m);
    mt = grp * g.group_m + i % rows;
    nt = i / rows;
}

// Rounds one chunk of accumulator columns of a row (v) to the BOX / 4 output words (w) of that row:
// BOX / 4 fp32 columns, or BOX / 2 columns packed two bfloat16 to a word.
template <int BOX, bool F32>
__device__ __forceinline__ void round_chunk(const uint32_t* v, uint32_t* w, const GemmArgs& g, const int64_t col0) {
    constexpr int W = BOX / 4;
    const float* bp = reinterpret_cast<const float*>(g.bias);
    if (F32) {
#pragma unroll
        for (int i = 0; i < W; ++i) {
            uint32_t b = round_out_bits(v[i], g.rnd);
            if (bp) b = round_out_bits(__float_as_uint(__uint_as_float(b) + __ldg(bp + min(col0 + i, g.N - 1))), g.rnd);
            w[i] = b;
        }
    } else if (g.epi_kind == 0) {              // half away: add half an ulp of bf16, keep the upper halves
#pragma unroll
        for (int i = 0; i < W; ++i) w[i] = __byte_perm(v[2 * i] + 0x8000u, v[2 * i + 1] + 0x8000u, 0x7632);
    } else if (g.epi_kind == 1) {              // toward zero
#pragma unroll
        for (int i = 0; i < W; ++i) w[i] = __byte_perm(v[2 * i], v[2 * i + 1], 0x7632);
    } else if (g.epi_kind == 2) {              // half even: the hardware conversion
#pragma unroll
        for (int i = 0; i < W; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(v[2 * i]), __uint_as_float(v[2 * i + 1]));
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
    } else {
#pragma unroll
        for (int i = 0; i < W; ++i) {
            uint32_t b0 = round_out_bits(v[2 * i], g.rnd);
            uint32_t b1 = round_out_bits(v[2 * i + 1], g.rnd);
            if (bp) {
                b0 = round_out_bits(__float_as_uint(__uint_as_float(b0) + __ldg(bp + min(col0 + 2 * i, g.N - 1))), g.rnd);
                b1 = round_out_bits(__float_as_uint(__uint_as_float(b1) + __ldg(bp + min(col0 + 2 * i + 1, g.N - 1))), g.rnd);
            }
            const __nv_bfloat162 h = __floats2bfloat162_rn(__uint_as_float(b0), __uint_as_float(b1));
            w[i] = *reinterpret_cast<const uint32_t*>(&h);
        }
    }
}

// One epilogue warp's share of an accumulator tile: kCols columns of its 32 tensor-memory lanes,
// starting at tensor-memory address `taddr` = column `first_col` of the tile.  The columns are
// drained in chunks of one output box (32 rows x BOX bytes): tcgen05.ld -> rounding -> swizzled
// staging buffer -> TMA store (which clips ragged M / N edges), or plain stores when the row
// pitch is not a multiple of 16 bytes.  The staging buffers of a warp form a ring of NBUF boxes
// (`ring` counts boxes across tiles); a box is rewritten once the bulk store issued NBUF boxes
// earlier has read it.  `after_first` runs when the first 32 columns have left tensor memory.
template <int kCols, int BOX, int NBUF, bool F32, typename AfterFirst>
__device__ __forceinline__ void drain_tile(const uint32_t taddr, const int first_col, const int lane, const uint32_t stg,
                                           uint32_t& ring, const GemmArgs& g, const CUtensorMap* tmap_c,
                                           const int64_t row0, const int64_t row0_dest, const int64_t tile_col0,
                                           const int64_t bi, AfterFirst after_first) {
    constexpr int CC = F32 ? BOX / 4 : BOX / 2;      // accumulator columns per chunk
    constexpr int W = BOX / 4;                       // output words per row and chunk
    static_assert(CC == 16 || CC == 32 || CC == 64, "chunk width");
#pragma unroll 1
    for (int c = 0; c < kCols; c += CC) {
        uint32_t v[CC];
        if constexpr (CC == 16) {
            ptx::tmem_ld_32x32b_x16(taddr + c, v);
        } else {
#pragma unroll
            for (int j = 0; j < CC; j += 32) ptx::tmem_ld_32x32b_x32(taddr + c + j, v + j);
        }
        ptx::tmem_ld_wait();
        if (c < 32 && c + CC >= 32) after_first();                // columns 0..31 have left tensor memory
        const int64_t col0 = tile_col0 + first_col + c;
        if (row0 >= g.M || col0 >= g.N) continue;                 // whole box outside the result (warp-uniform)
        uint32_t w[W];
        round_chunk<BOX, F32>(v, w, g, col0);
        if (g.c_tma) {
            const uint32_t buf = stg + (ring % NBUF) * (32 * BOX);
            ++ring;
            if (lane == 0) ptx::bulk_wait_read<NBUF - 1>();      // this box's previous store has read it
            __syncwarp();
#pragma unroll
            for (int q = 0; q < BOX / 16; ++q) {
                const int sw = BOX == 128 ? (q ^ (lane & 7)) : (q ^ ((lane >> 1) & 3));
                ptx::st_shared_v4(buf + lane * BOX + (sw << 4), w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
            }
            ptx::fence_proxy_async();
            __syncwarp();
            if (lane == 0) {
                ptx::tma_store_3d(tmap_c, buf, (int)col0, (int)row0_dest, (int)bi);
                ptx::bulk_commit();
            }
        } else if (row0 + lane < g.M) {
            const int64_t off = (bi * g.M + row0 + lane) * g.N + col0;
#pragma unroll
            for (int i = 0; i < W; ++i) {
                if (F32) {
                    if (col0 + i < g.N) reinterpret_cast<uint32_t*>(g.c)[off + i] = w[i];
                } else {
                    if (col0 + 2 * i < g.N) reinterpret_cast<uint16_t*>(g.c)[off + 2 * i] = (uint16_t)w[i];
                    if (col0 + 2 * i + 1 < g.N) reinterpret_cast<uint16_t*>(g.c)[off + 2 * i + 1] = (uint16_t)(w[i] >> 16);
                }
            }
        }
    }
}

// Tensor-memory columns.  Two accumulators of 256 columns fill the 512 columns completely, so the
// scale columns of the tile being computed (4 for A, BN / 32 for B, twice that when the K blocks
// alternate between two sets) are parked in the first 32 columns of the OTHER accumulator: the
// previous tile's epilogue reads those columns first and hands them back (`sf_free`) long before
// it has drained the rest, so the next tile's MMAs start almost at once.
constexpr uint32_t kTmemCols = 512;
// K blocks alternate between two sets of scale columns so that the copy of block j + 1's scales
// need not wait for the MMAs of block j to have read theirs.
constexpr uint32_t kSfSets = 2;
constexpr uint32_t kSfSetCols = 16;

template <int BN, int STAGES, int ACC_BUFS, int BOX, int NBUF>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_mx_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
               const __grid_constant__ OutMaps tmaps_c, const GemmArgs g) {
    using S = GemmSmem<BN, STAGES, BOX, NBUF>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBarOff);
    // barrier indices
    uint64_t* full = bars;                       // [STAGES]
    uint64_t* empty = bars + STAGES;             // [STAGES]
    uint64_t* acc_full = bars + 2 * STAGES;      // [ACC_BUFS]
    uint64_t* acc_empty = acc_full + ACC_BUFS;   // [ACC_BUFS]
    uint64_t* sf_free = acc_empty + ACC_BUFS;    // [ACC_BUFS]  (kSfSwap only)
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sf_free + ACC_BUFS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    constexpr uint32_t kAccCols = BN * ACC_BUFS;
    constexpr bool kSfSwap = kAccCols + kSfSets * kSfSetCols > kTmemCols;
    static_assert(!kSfSwap || (ACC_BUFS == 2 && kAccCols == kTmemCols), "scale columns need a home");
    static_assert(4 + BN / 32 <= kSfSetCols, "scale set width");

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { ptx::mbar_init(ptx::smem_u32(&full[s]), 1); ptx::mbar_init(ptx::smem_u32(&empty[s]), 1); }
        for (int b = 0; b < ACC_BUFS; ++b) {
            ptx::mbar_init(ptx::smem_u32(&acc_full[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&acc_empty[b]), kEpiWarps);
            ptx::mbar_init(ptx::smem_u32(&sf_free[b]), 4);               // the four warps that own columns 0..31
        }
        *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(tmem_slot), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t tiles_per_batch = g.m_tiles * g.n_tiles;
    const int64_t total_tiles = tiles_per_batch * g.batch;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (ptx::elect_one()) {
            ptx::prefetch_tmap(&tmap_a);
            ptx::prefetch_tmap(&tmap_b);
            uint32_t it = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x) {
                int64_t bi, mt, nt;
                tile_coords(t, g, tiles_per_batch, bi, mt, nt);
                for (int64_t kb = 0; kb < g.k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (it >= (uint32_t)STAGES && !ptx::mbar_wait(ptx::smem_u32(&empty[s]), ph ^ 1, abort_flag)) { ok = false; break; }
                    uint8_t* st = smem + (size_t)s * S::kStage;
                    const uint32_t bar = ptx::smem_u32(&full[s]);
                    ptx::mbar_expect_tx(bar, S::kStage);
                    ptx::tma_load_3d(ptx::smem_u32(st), &tmap_a, bar, (int)(kb * kBK), (int)(mt * kBM), (int)bi);
                    ptx::tma_load_3d(ptx::smem_u32(st + S::kA), &tmap_b, bar, (int)(kb * kBK), (int)(nt * BN), (int)bi);
                    ptx::bulk_load(ptx::smem_u32(st + S::kA + S::kB),
                                   g.sfa + ((bi * g.sfa_rows128 + mt) * g.k_blocks + kb) * kSfChunk, kSfChunk, bar);
#pragma unroll
                    for (int j = 0; j < BN / 128; ++j)
                        ptx::bulk_load(ptx::smem_u32(st + S::kA + S::kB + S::kSFA + j * kSfChunk),
                                       g.sfb + ((bi * g.sfb_rows128 + nt * (BN / 128) + j) * g.k_blocks + kb) * kSfChunk,
                                       kSfChunk, bar);
                }
            }
            if (!ok) {
                // drain: give copies already in flight a bounded time to land
                for (int s = 0; s < STAGES; ++s)
                    for (uint32_t i = 0; i < 4096 && !ptx::mbar_try_wait(ptx::smem_u32(&full[s]), 0) &&
                                         !ptx::mbar_try_wait(ptx::smem_u32(&full[s]), 1); ++i) __nanosleep(64);
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (ptx::elect_one()) {
            uint32_t it = 0, tile_i = 0;
            bool ok = true;
            for (int64_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_i) {
                const int buf = tile_i % ACC_BUFS;
                const uint32_t acc_ph = (tile_i / ACC_BUFS) & 1;
                if (tile_i >= (uint32_t)ACC_BUFS && !ptx::mbar_wait(ptx::smem_u32(&acc_empty[buf]), acc_ph ^ 1, abort_flag)) { ok = false; break; }
                if (kSfSwap && tile_i >= 1 &&
                    !ptx::mbar_wait(ptx::smem_u32(&sf_free[buf ^ 1]), ((tile_i - 1) / ACC_BUFS) & 1, abort_flag)) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)buf * BN;
                const uint32_t sf_home = tmem_base + (kSfSwap ? (uint32_t)(buf ^ 1) * BN : kAccCols);
                for (int64_t kb = 0; kb < g.k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!ptx::mbar_wait(ptx::smem_u32(&full[s]), ph, abort_flag)) { ok = false; break; }
                    ptx::tc_fence_after();
                    uint8_t* st = smem + (size_t)s * S::kStage;
                    const uint32_t a_addr = ptx::smem_u32(st);
                    const uint32_t b_addr = ptx::smem_u32(st + S::kA);
                    const uint32_t sfa_addr = ptx::smem_u32(st + S::kA + S::kB);
                    const uint32_t sfb_addr = sfa_addr + S::kSFA;
                    const uint32_t sfa_col = sf_home + (it % kSfSets) * kSfSetCols;
                    const uint32_t sfb_col = sfa_col + 4;
                    // scales: 32 rows x 16 bytes per chunk, 8-row groups 128 bytes apart, no swizzle
                    ptx::tc_cp_32x128b_warpx4(sfa_col, ptx::smem_desc(sfa_addr, 0, 128, 0));
#pragma unroll
                    for (int j = 0; j < BN / 128; ++j)
                        ptx::tc_cp_32x128b_warpx4(sfb_col + 4 * j, ptx::smem_desc(sfb_addr + j * kSfChunk, 0, 128, 0));
#pragma unroll
                    for (int k = 0; k < kBK / 32; ++k) {
                        // K-major, 128-byte swizzle: 8-row groups 1024 bytes apart; a K step of
                        // 32 elements moves the start address by 32 bytes inside the swizzle atom
                        const uint64_t ad = ptx::smem_desc(a_addr + 32 * k, 0, 1024, 2);
                        const uint64_t bd = ptx::smem_desc(b_addr + 32 * k, 0, 1024, 2);
                        const uint32_t id = g.idesc | ((uint32_t)k << 4) | ((uint32_t)k << 29);
                        ptx::tc_mma_mxf8f6f4(d_tmem, ad, bd, id, sfa_col | ((uint32_t)k << 30),
                                             sfb_col | ((uint32_t)k << 30), (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    ptx::tc_commit(ptx::smem_u32(&empty[s]));        // stage reusable once these MMAs retire
                }
                if (ok) ptx::tc_commit(ptx::smem_u32(&acc_full[buf]));
            }
        }
    } else {
        // ---------------- epilogue warps ----------------
        // Warp (2 + e) drains lane quarter (warp & 3), column half (e >> 2) of the accumulator.
        const int e = warp - 2;
        const int q = warp & 3;                               // the tensor-memory lane quarter this warp may read
        const int half = e >> 2;
        const uint32_t stg = ptx::smem_u32(smem + S::kStgOff + e * S::kStgWarp);
        constexpr int kCols = BN / 2;
        uint32_t tile_i = 0, ring = 0;
        bool ok = true;
        for (int64_t t = blockIdx.x; t < total_tiles && ok; t += gridDim.x, ++tile_i) {
            const int buf = tile_i % ACC_BUFS;
            const uint32_t acc_ph = (tile_i / ACC_BUFS) & 1;
            int64_t bi, mt, nt;
            tile_coords(t, g, tiles_per_batch, bi, mt, nt);
            if (!ptx::mbar_wait(ptx::smem_u32(&acc_full[buf]), acc_ph, abort_flag)) { ok = false; break; }
            ptx::tc_fence_after();
            const int64_t row0 = mt * kBM + q * 32;
            // destination of this tile's rows (128-row tiles never straddle destinations)
            const int64_t dest = g.rows_per_dest > 0 ? row0 / g.rows_per_dest : 0;
            const int64_t row0_dest = row0 - dest * g.rows_per_dest;
            const CUtensorMap* tmap_c = &tmaps_c.m[dest < kMaxDests ? dest : 0];
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)buf * BN + half * kCols;
            auto after_first = [&]() {
                if (kSfSwap && half == 0) {                   // columns 0..31 are out: the next tile's scales go there
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&sf_free[buf]));
                }
            };
            if (g.out_dtype == DT_F32)
                drain_tile<kCols, BOX, NBUF, true>(taddr, half * kCols, lane, stg, ring, g, tmap_c, row0, row0_dest, nt * BN, bi, after_first);
            else
                drain_tile<kCols, BOX, NBUF, false>(taddr, half * kCols, lane, stg, ring, g, tmap_c, row0, row0_dest, nt * BN, bi, after_first);
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&acc_empty[buf]));
        }
        if (lane == 0) ptx::bulk_wait_all();
    }

    // ---------------- teardown ----------------
    ptx::tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(g.status, MXQ_ERR_DEVICE);
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------
// CTA-pair kernel (cta_group::2): two CTAs of a cluster share one 256 x 256
// tile.  Each CTA stages its own 128 rows of A, its own 128-row half of the B
// tile and the scales it needs (its rows of A, all 256 columns of B), so a K
// block costs 33.5 KB of shared-memory fill per SM instead of 49.5 KB; the even
// CTA issues tcgen05.cp / tcgen05.mma for both, and every CTA drains the 128
// accumulator rows held in its own tensor memory.  Two accumulators alternate
// (the scale columns parked in the idle one, as above), so the drain of a tile
// runs under the main loop of the next.  Barriers: `full` lives in the even
// CTA and counts the bytes of both CTAs' loads; `empty` and `acc_full` exist in
// both CTAs and are signalled together by a multicast commit; `acc_empty` and
// `sf_free` live in the even CTA and collect the epilogue warps of both.
// No load is multicast.  All waits are bounded as in the single-CTA kernel.
// ---------------------------------------------------------------------------
constexpr int kPairBN = 256;
template <int STAGES, int BOX, int NBUF>
struct PairSmem {
    static constexpr int kA = kBM * kBK;                   // this CTA's rows of A
    static constexpr int kB = 128 * kBK;                   // this CTA's half of the B tile
    static constexpr int kAB = kA + kB;
    static constexpr int kSF = 3 * kSfChunk;               // scales: A (own rows) + B (256 columns)
    static constexpr int kStageBytes = kAB + kSF;          // bytes one CTA loads per K block
    static constexpr int kSfOff = STAGES * kAB;
    static constexpr int kStgOff = (kSfOff + STAGES * kSF + 1023) / 1024 * 1024;
    static constexpr int kStgWarp = 32 * BOX * NBUF;
    static constexpr int kBarOff = kStgOff + kEpiWarps * kStgWarp;
    static constexpr int kTotal = kBarOff + 256 + 1024;
};

template <int STAGES, int BOX, int NBUF>
__global__ void __launch_bounds__(kGemmThreads, 1)
gemm_mx_pair_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b,
                    const __grid_constant__ CUtensorMap tmap_sfa, const __grid_constant__ CUtensorMap tmap_sfb,
                    const __grid_constant__ OutMaps tmaps_c, const GemmArgs g) {
    using S = PairSmem<STAGES, BOX, NBUF>;
    constexpr int BN = kPairBN;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + S::kBarOff);
    uint64_t* full = bars;                       // [STAGES]  used in the even CTA
    uint64_t* empty = bars + STAGES;             // [STAGES]  one per CTA
    uint64_t* acc_full = bars + 2 * STAGES;      // [2]  one per CTA
    uint64_t* acc_empty = acc_full + 2;          // [2]  used in the even CTA
    uint64_t* sf_free = acc_empty + 2;           // [2]  used in the even CTA
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(sf_free + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const uint32_t rank = ptx::cluster_ctarank();             // 0 = even CTA (issues the MMAs)

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) { ptx::mbar_init(ptx::smem_u32(&full[s]), 1); ptx::mbar_init(ptx::smem_u32(&empty[s]), 1); }
        for (int b = 0; b < 2; ++b) {
            ptx::mbar_init(ptx::smem_u32(&acc_full[b]), 1);
            ptx::mbar_init(ptx::smem_u32(&acc_empty[b]), 2 * kEpiWarps);
            ptx::mbar_init(ptx::smem_u32(&sf_free[b]), 2 * 4);           // the warps of both CTAs that own columns 0..31
        }
        *abort_flag = 0;
        ptx::fence_mbar_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(tmem_slot), kTmemCols);
        ptx::tmem_relinquish_pair();
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_arrive();                                    // both CTAs' barriers exist before anyone signals them
    ptx::cluster_wait();
    ptx::tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const int64_t tiles_per_batch = g.m_tiles * g.n_tiles;    // 256 x 256 tiles
    const int64_t total_tiles = tiles_per_batch * g.batch;
    const int64_t pair = blockIdx.x >> 1, n_pairs = gridDim.x >> 1;

    if (warp == 0) {
        // ---------------- TMA producer (one per CTA) ----------------
        if (ptx::elect_one()) {
            ptx::prefetch_tmap(&tmap_a);
            ptx::prefetch_tmap(&tmap_b);
            ptx::prefetch_tmap(&tmap_sfa);
            ptx::prefetch_tmap(&tmap_sfb);
            uint32_t it = 0;
            bool ok = true;
            for (int64_t t = pair; t < total_tiles && ok; t += n_pairs) {
                int64_t bi, mt2, nt;
                tile_coords(t, g, tiles_per_batch, bi, mt2, nt);
                const int64_t mt = 2 * mt2 + rank;             // this CTA's 128-row tile
                for (int64_t kb = 0; kb < g.k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (it >= (uint32_t)STAGES && !ptx::mbar_wait(ptx::smem_u32(&empty[s]), ph ^ 1, abort_flag)) { ok = false; break; }
                    if (rank == 0) ptx::mbar_expect_tx(ptx::smem_u32(&full[s]), 2 * S::kStageBytes);
                    const uint32_t bar = ptx::mapa(ptx::smem_u32(&full[s]), 0);
                    const uint32_t ab = ptx::smem_u32(smem + (size_t)s * S::kAB);
                    const uint32_t sf = ptx::smem_u32(smem + S::kSfOff + (size_t)s * S::kSF);
                                        ptx::tma_load_3d_pair(ab, &tmap_a, bar, (int)(kb * kBK), (int)(mt * kBM), (int)bi);
                    ptx::tma_load_3d_pair(ab + S::kA, &tmap_b, bar, (int)(kb * kBK), (int)(nt * BN + rank * 128), (int)bi);
                    ptx::tma_load_4d_pair(sf, &tmap_sfa, bar, 0, (int)kb, (int)mt, (int)bi);
                    ptx::tma_load_4d_pair(sf + kSfChunk, &tmap_sfb, bar, 0, (int)kb, (int)(nt * 2), (int)bi);
                    ptx::tma_load_4d_pair(sf + 2 * kSfChunk, &tmap_sfb, bar, 0, (int)kb, (int)(nt * 2 + 1), (int)bi);
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer (even CTA only) ----------------
        if (rank == 0 && ptx::elect_one()) {
            uint32_t it = 0, tile_i = 0;
            bool ok = true;
            for (int64_t t = pair; t < total_tiles && ok; t += n_pairs, ++tile_i) {
                const uint32_t buf = tile_i & 1;
                const uint32_t acc_ph = (tile_i >> 1) & 1;
                if (tile_i >= 2 && !ptx::mbar_wait(ptx::smem_u32(&acc_empty[buf]), acc_ph ^ 1, abort_flag)) { ok = false; break; }
                if (tile_i >= 1 && !ptx::mbar_wait(ptx::smem_u32(&sf_free[buf ^ 1]), ((tile_i - 1) >> 1) & 1, abort_flag)) { ok = false; break; }
                ptx::tc_fence_after();
                const uint32_t d_tmem = tmem_base + buf * BN;
                const uint32_t sf_home = tmem_base + (buf ^ 1) * BN;
                for (int64_t kb = 0; kb < g.k_blocks; ++kb, ++it) {
                    const int s = it % STAGES;
                    const uint32_t ph = (it / STAGES) & 1;
                    if (!ptx::mbar_wait(ptx::smem_u32(&full[s]), ph, abort_flag)) { ok = false; break; }
                    ptx::tc_fence_after();
                    const uint32_t a_addr = ptx::smem_u32(smem + (size_t)s * S::kAB);
                    const uint32_t b_addr = a_addr + S::kA;
                    const uint32_t sf_addr = ptx::smem_u32(smem + S::kSfOff + (size_t)s * S::kSF);
                    const uint32_t sfa_col = sf_home + (it % kSfSets) * kSfSetCols;
                    const uint32_t sfb_col = sfa_col + 4;
                    ptx::tc_cp_32x128b_warpx4_pair(sfa_col, ptx::smem_desc(sf_addr, 0, 128, 0));
                    ptx::tc_cp_32x128b_warpx4_pair(sfb_col, ptx::smem_desc(sf_addr + kSfChunk, 0, 128, 0));
                    ptx::tc_cp_32x128b_warpx4_pair(sfb_col + 4, ptx::smem_desc(sf_addr + 2 * kSfChunk, 0, 128, 0));
#pragma unroll
                    for (int k = 0; k < kBK / 32; ++k) {
                        const uint64_t ad = ptx::smem_desc(a_addr + 32 * k, 0, 1024, 2);
                        const uint64_t bd = ptx::smem_desc(b_addr + 32 * k, 0, 1024, 2);
                        const uint32_t id = g.idesc | ((uint32_t)k << 4) | ((uint32_t)k << 29);
                        ptx::tc_mma_mxf8f6f4_pair(d_tmem, ad, bd, id, sfa_col | ((uint32_t)k << 30),
                                                  sfb_col | ((uint32_t)k << 30), (kb > 0 || k > 0) ? 1u : 0u);
                    }
                    ptx::tc_commit_pair(ptx::smem_u32(&empty[s]), 3);      // both CTAs may refill the stage
                }
                if (ok) ptx::tc_commit_pair(ptx::smem_u32(&acc_full[buf]), 3);
            }
        }
    } else {
        // ---------------- epilogue warps (both CTAs, 128 rows each) ----------------
        const int e = warp - 2;
        const int q = warp & 3;
        const int half = e >> 2;
        const uint32_t stg = ptx::smem_u32(smem + S::kStgOff + e * S::kStgWarp);
        constexpr int kCols = BN / 2;
        uint32_t tile_i = 0, ring = 0;
        bool ok = true;
        for (int64_t t = pair; t < total_tiles && ok; t += n_pairs, ++tile_i) {
            const uint32_t buf = tile_i & 1;
            int64_t bi, mt2, nt;
            tile_coords(t, g, tiles_per_batch, bi, mt2, nt);
            if (!ptx::mbar_wait(ptx::smem_u32(&acc_full[buf]), (tile_i >> 1) & 1, abort_flag)) { ok = false; break; }
            ptx::tc_fence_after();
            const int64_t row0 = (2 * mt2 + rank) * kBM + q * 32;
            const int64_t dest = g.rows_per_dest > 0 ? row0 / g.rows_per_dest : 0;
            const int64_t row0_dest = row0 - dest * g.rows_per_dest;
            const CUtensorMap* tmap_c = &tmaps_c.m[dest < kMaxDests ? dest : 0];
            const uint32_t taddr = tmem_base + ((uint32_t)(q * 32) << 16) + buf * BN + half * kCols;
            auto after_first = [&]() {
                if (half == 0) {
                    ptx::tc_fence_before();
                    __syncwarp();
                    if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa(ptx::smem_u32(&sf_free[buf]), 0));
                }
            };
            if (g.out_dtype == DT_F32)
                drain_tile<kCols, BOX, NBUF, true>(taddr, half * kCols, lane, stg, ring, g, tmap_c, row0, row0_dest, nt * BN, bi, after_first);
            else
                drain_tile<kCols, BOX, NBUF, false>(taddr, half * kCols, lane, stg, ring, g, tmap_c, row0, row0_dest, nt * BN, bi, after_first);
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(ptx::mapa(ptx::smem_u32(&acc_empty[buf]), 0));
        }
        if (lane == 0) ptx::bulk_wait_all();
    }

    // ---------------- teardown ----------------
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_arrive();                                    // the partner no longer touches this CTA's memory
    ptx::cluster_wait();
    if (threadIdx.x == 0 && *abort_flag) atomicExch(g.status, MXQ_ERR_DEVICE);
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, kTmemCols);
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
// [batch, rows, K] bytes, K contiguous; box = 128 bytes of K x box_rows rows
static int make_operand_map(CUtensorMap* m, const void* base, int64_t batch, int64_t rows, int64_t K, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return MXQ_ERR_CUDA;
    cuuint64_t dims[3] = {(cuuint64_t)K, (cuuint64_t)rows, (cuuint64_t)batch};
    cuuint64_t strides[2] = {(cuuint64_t)K, (cuuint64_t)(K * rows)};
    cuuint32_t box[3] = {(cuuint32_t)kBK, (cuuint32_t)box_rows, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT8, 3, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MXQ_OK : MXQ_ERR_CUDA;
}

static int* device_status_word() {
    // one status word per device, allocated on first use and kept until exit
    static int* words[64] = {nullptr};
    static std::mutex mu;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!words[dev]) {
        int* w = nullptr;
        if (cudaMalloc(&w, 64) != cudaSuccess) { cudaGetLastError(); return nullptr; }
        if (cudaMemset(w, 0, 64) != cudaSuccess) { cudaFree(w); return nullptr; }
        words[dev] = w;
    }
    return words[dev];
}

// C [batch, M, N]: box = box_bytes (64 or 128) of a row x 32 rows, swizzle of the same width
static int make_output_map(CUtensorMap* m, void* base, int64_t batch, int64_t M, int64_t N, bool f32, int box_bytes) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return MXQ_ERR_CUDA;
    const cuuint64_t es = f32 ? 4 : 2;
    cuuint64_t dims[3] = {(cuuint64_t)N, (cuuint64_t)M, (cuuint64_t)batch};
    cuuint64_t strides[2] = {(cuuint64_t)N * es, (cuuint64_t)N * M * es};
    cuuint32_t box[3] = {(cuuint32_t)(box_bytes / es), 32, 1};
    cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = fn(m, f32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, base, dims,
                          strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          box_bytes == 128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_64B,
                          CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MXQ_OK : MXQ_ERR_CUDA;
}

// E8M0 scales as a 4-D tensor of 512-byte chunks: [batch][128-row chunk][K block][128 words]
static int make_sf_map(CUtensorMap* m, const void* base, int64_t batch, int64_t rows128, int64_t k_blocks) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return MXQ_ERR_CUDA;
    cuuint64_t dims[4] = {128, (cuuint64_t)k_blocks, (cuuint64_t)rows128, (cuuint64_t)batch};
    cuuint64_t strides[3] = {(cuuint64_t)kSfChunk, (cuuint64_t)kSfChunk * k_blocks, (cuuint64_t)kSfChunk * k_blocks * rows128};
    cuuint32_t box[4] = {128, 1, 1, 1};
    cuuint32_t estr[4] = {1, 1, 1, 1};
    const CUresult r = fn(m, CU_TENSOR_MAP_DATA_TYPE_UINT32, 4, const_cast<void*>(base), dims, strides, box, estr,
                          CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? MXQ_OK : MXQ_ERR_CUDA;
}

template <int STAGES, int BOX, int NBUF>
static int launch_gemm_pair(const CUtensorMap& ta, const CUtensorMap& tb, const CUtensorMap& tsa, const CUtensorMap& tsb,
                            const OutMaps& tc, const GemmArgs& g, cudaStream_t st) {
    using S = PairSmem<STAGES, BOX, NBUF>;
    static_assert(S::kTotal <= 232448, "shared memory of the pair kernel");
    auto kern = gemm_mx_pair_kernel<STAGES, BOX, NBUF>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) != cudaSuccess)
        return MXQ_ERR_CUDA;
    const int64_t tiles = g.m_tiles * g.n_tiles * g.batch;
    const int pairs = (int)std::min<int64_t>(tiles, std::max(gemm_sms() / 2, 1));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = S::kTotal;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2; attr[0].val.clusterDim.y = 1; attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    if (cudaLaunchKernelEx(&cfg, kern, ta, tb, tsa, tsb, tc, g) != cudaSuccess) { cudaGetLastError(); return MXQ_ERR_CUDA; }
    return check_launch();
}

template <int BN, int STAGES, int ACC_BUFS, int BOX, int NBUF>
static int launch_gemm(const CUtensorMap& ta, const CUtensorMap& tb, const OutMaps& tc, const GemmArgs& g,
                       cudaStream_t st) {
    using S = GemmSmem<BN, STAGES, BOX, NBUF>;
    static_assert(S::kTotal <= 232448, "shared memory of the single-CTA kernel");
    auto kern = gemm_mx_kernel<BN, STAGES, ACC_BUFS, BOX, NBUF>;
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::kTotal) != cudaSuccess)
        return MXQ_ERR_CUDA;
    const int64_t tiles = g.m_tiles * g.n_tiles * g.batch;
    const int grid = (int)std::min<int64_t>(tiles, gemm_sms());
    kern<<<grid, kGemmThreads, S::kTotal, st>>>(ta, tb, tc, g);
    return check_launch();
}

}  // namespace mxq

extern "C" int64_t mxq_sf_bytes(int64_t batch, int64_t rows, int64_t K) {
    if (batch < 0 || rows < 0 || K < 0) return -1;
    return batch * ((rows + 127) / 128) * ((K + 127) / 128) * 512;
}

namespace mxq {
// The GEMM with the device status word supplied by the caller (4 bytes of
// device memory the kernel writes MXQ_ERR_DEVICE to when it gives up on a wait).
int gemm_mx_with_status(const void* a_codes, const void* a_scales, const void* b_codes, const void* b_scales,
                        void* c, int64_t batch, int64_t M, int64_t N, int64_t K, int a_fmt, int b_fmt,
                        int out_dtype, int out_bfloat_bits, int out_round, const void* bias, int tile_n,
                        int* status_word, void* stream, void* const* dests, int n_dests, int64_t rows_per_dest) {
    if (n_dests > 0) {
        if (!dests || n_dests > kMaxDests || rows_per_dest <= 0 || rows_per_dest % kBM != 0 || batch != 1 ||
            M > n_dests * rows_per_dest)
            return MXQ_ERR_BAD_ARG;
        for (int d = 0; d < n_dests; ++d)
            if (!dests[d] || !aligned16(dests[d])) return MXQ_ERR_BAD_ARG;
        c = dests[0];
    }
    if (batch < 0 || M < 0 || N < 0 || K < 0) return MXQ_ERR_BAD_ARG;
    if (batch == 0 || M == 0 || N == 0) return MXQ_OK;
    if (!a_codes || !a_scales || !b_codes || !b_scales || !c) return MXQ_ERR_BAD_ARG;
    // K: whole 32-element blocks and a 16-byte row pitch.  A last K block shorter than 128 is zero-filled
    // by the tiled loads; its unused scale bytes must be finite (the quantizer's buffers are zeroed there).
    if (K == 0 || K % 32 != 0) return MXQ_ERR_UNSUPPORTED;
    if (a_fmt < 0 || a_fmt > 1 || b_fmt < 0 || b_fmt > 1) return MXQ_ERR_BAD_ARG;
    if (out_dtype != MXQ_F32 && out_dtype != MXQ_BF16) return MXQ_ERR_BAD_ARG;
    if (out_round < -1 || out_round > MXQ_ROUND_EVEN) return MXQ_ERR_BAD_ARG;
    if (out_bfloat_bits != 0 && (out_bfloat_bits < 10 || out_bfloat_bits > 32)) return MXQ_ERR_BAD_ARG;
    if (!aligned16(a_codes) || !aligned16(b_codes) || !aligned16(a_scales) || !aligned16(b_scales) || !aligned16(c))
        return MXQ_ERR_ALIGN;
    if (batch > 0x7fffffff || M > 0x7fffffff || N > 0x7fffffff || K > 0x7fffffff) return MXQ_ERR_TOO_LARGE;
    int bn = (tile_n == 128 || tile_n == 256) ? tile_n : (N > 128 ? 256 : 128);
    // a 256-wide tile reads two 128-row scale chunks per K block; fall back to 128-wide
    // tiles when the scale buffer of B has an odd number of row chunks
    if (bn == 256 && ((N + 127) / 128) % 2 != 0) bn = 128;
    GemmArgs g;
    g.sfa = (const uint8_t*)a_scales; g.sfb = (const uint8_t*)b_scales; g.c = c; g.bias = bias;
    g.status = status_word;
    if (!g.status) return MXQ_ERR_CUDA;
    g.M = M; g.N = N; g.K = K; g.batch = batch;
    g.group_m = kGroupM;
    g.m_tiles = (M + kBM - 1) / kBM; g.n_tiles = (N + bn - 1) / bn; g.k_blocks = (K + kBK - 1) / kBK;
    g.sfa_rows128 = (M + 127) / 128; g.sfb_rows128 = (N + 127) / 128;
    g.idesc = ptx::idesc_block_scaled(a_fmt, b_fmt, kBM, bn);
    g.out_dtype = out_dtype;
    const bool rounds = out_bfloat_bits >= 10 && out_bfloat_bits < 32 && out_round >= 0;
    const uint32_t drop = rounds ? (uint32_t)(32 - out_bfloat_bits) : 0;
    const uint32_t mask = rounds ? ((1u << drop) - 1u) : 0u;
    g.rnd.drop = drop;
    g.rnd.keep = ~mask;
    g.rnd.even_on = (rounds && out_round == MXQ_ROUND_EVEN) ? 1u : 0u;
    g.rnd.add = !rounds ? 0u : (out_round == MXQ_ROUND_NEAREST ? (1u << (drop - 1)) : (out_round == MXQ_ROUND_EVEN ? (mask >> 1) : 0u));
    g.epi_kind = (out_dtype == MXQ_BF16 && rounds && drop == 16 && !bias) ? out_round : 3;
    g_launch_count[0].fetch_add(1, std::memory_order_relaxed);
    CUtensorMap ta, tb;
    int rc = make_operand_map(&ta, a_codes, batch, M, K, kBM);
    if (rc) return rc;
    rc = make_operand_map(&tb, b_codes, batch, N, K, bn);
    if (rc) return rc;
    const int64_t es = out_dtype == MXQ_F32 ? 4 : 2;
    g.c_tma = (N * es) % 16 == 0;
    g.rows_per_dest = n_dests > 0 ? rows_per_dest : 0;
    if (n_dests > 0 && !g.c_tma) return MXQ_ERR_UNSUPPORTED;          // destinations are written by TMA stores only
    // Engine.  CTA pairs on 256 x 256 tiles when the problem gives every SM pair a tile and has a long
    // K loop; otherwise single CTAs on 128 x 256 tiles (a short K loop makes the kernel store-bound:
    // fewer operand stages, wide output boxes and a deeper staging ring), or 128 x 128 for narrow N.
    const int64_t tiles2 = ((M + 255) / 256) * ((N + 255) / 256) * batch;
    const bool pair = tiles2 >= sm_count() / 2 && M >= 256 && N >= 256 && K >= 1024 && g.c_tma;
    const bool short_k = !pair && bn == 256 && K <= 512;
    const int box_bytes = pair ? MXQ_PAIR_BOX : (short_k ? 128 : 64);
    OutMaps tc;
    for (int d = 0; d < kMaxDests; ++d) tc.m[d] = ta;                  // placeholders, never dereferenced
    if (n_dests > 0) {
        for (int d = 0; d < n_dests; ++d) {
            const int64_t rows = std::min<int64_t>(rows_per_dest, M - d * rows_per_dest);   // the last one may be ragged
            if (rows <= 0) break;
            rc = make_output_map(&tc.m[d], dests[d], 1, rows, N, out_dtype == MXQ_F32, box_bytes);
            if (rc) return rc;
        }
    } else if (g.c_tma) {
        rc = make_output_map(&tc.m[0], c, batch, M, N, out_dtype == MXQ_F32, box_bytes);
        if (rc) return rc;
    }
    if (pair) {
        GemmArgs gp = g;
        gp.m_tiles = (M + 255) / 256;
        gp.n_tiles = (N + 255) / 256;
        gp.idesc = ptx::idesc_block_scaled(a_fmt, b_fmt, 256, 256);
        CUtensorMap tb2, tsa, tsb;
        rc = make_operand_map(&tb2, b_codes, batch, N, K, 128);
        if (rc) return rc;
        rc = make_sf_map(&tsa, a_scales, batch, g.sfa_rows128, g.k_blocks);
        if (rc) return rc;
        rc = make_sf_map(&tsb, b_scales, batch, g.sfb_rows128, g.k_blocks);
        if (rc) return rc;
        return launch_gemm_pair<MXQ_PAIR_STAGES, MXQ_PAIR_BOX, 1>(ta, tb2, tsa, tsb, tc, gp, (cudaStream_t)stream);
    }
    if (short_k) return launch_gemm<256, 3, 2, 128, 2>(ta, tb, tc, g, (cudaStream_t)stream);
    if (bn == 256) return launch_gemm<256, 4, 2, 64, 1>(ta, tb, tc, g, (cudaStream_t)stream);
    return launch_gemm<128, 6, 2, 64, 1>(ta, tb, tc, g, (cudaStream_t)stream);
}
}  // namespace mxq

extern "C" int mxq_gemm_mx(const void* a_codes, const void* a_scales, const void* b_codes, const void* b_scales,
                           void* c, int64_t batch, int64_t M, int64_t N, int64_t K, int a_fmt, int b_fmt,
                           int out_dtype, int out_bfloat_bits, int out_round, const void* bias, int tile_n,
                           void* stream) {
    if (batch < 0 || M < 0 || N < 0 || K < 0) return MXQ_ERR_BAD_ARG;
    if (batch == 0 || M == 0 || N == 0) return MXQ_OK;
    int* word = mxq::device_status_word();
    if (!word) return MXQ_ERR_CUDA;
    return mxq::gemm_mx_with_status(a_codes, a_scales, b_codes, b_scales, c, batch, M, N, K, a_fmt, b_fmt, out_dtype,
                                    out_bfloat_bits, out_round, bias, tile_n, word, stream, nullptr, 0, 0);
}

extern "C" int mxq_gemm_mx_scatter(const void* a_codes, const void* a_scales, const void* b_codes, const void* b_scales,
                                   void* const* dests, int n_dests, int64_t rows_per_dest, int64_t M, int64_t N,
                                   int64_t K, int a_fmt, int b_fmt, int out_dtype, int out_bfloat_bits, int out_round,
                                   int tile_n, void* stream) {
    if (M < 0 || N < 0 || K < 0 || n_dests <= 0) return MXQ_ERR_BAD_ARG;
    if (M == 0 || N == 0) return MXQ_OK;
    int* word = mxq::device_status_word();
    if (!word) return MXQ_ERR_CUDA;
    return mxq::gemm_mx_with_status(a_codes, a_scales, b_codes, b_scales, nullptr, 1, M, N, K, a_fmt, b_fmt, out_dtype,
                                    out_bfloat_bits, out_round, nullptr, tile_n, word, stream, dests, n_dests,
                                    rows_per_dest);
}

extern "C" int mxq_device_status(int clear) {
    int* w = mxq::device_status_word();
    if (!w) return MXQ_ERR_CUDA;
    int v = 0;
    if (cudaMemcpy(&v, w, sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) return MXQ_ERR_CUDA;
    if (clear && v != 0) cudaMemset(w, 0, sizeof(int));
    return v;
}
