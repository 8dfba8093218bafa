// Persistent, warp-specialised tcgen05 GEMM for sm_100a, with two front ends:
//
//   * plain / split-operand GEMM   C[M,N] = sum_s A_s[M,K] * B_s  (+bias, +residual)
//   * halo-aware implicit-GEMM 3x3 convolution on an H-strip in NHWC, whose A
//     tiles are gathered by TMA row by row from three sources: the fresh local
//     strip and the (stale) boundary rows of the strips above and below.
//
// Roles inside a CTA of 352 threads (one CTA per SM, tiles strided by grid; kEpiSub = 2):
//   warps 8, 10 TMA producers (A and B operand): fill a ring of {A 128x64, B BNx64} fp16 stages
//   warp 9      allocates tensor memory and issues tcgen05.mma (one lane)
//   warps 0..7  epilogue, kEpiSub warps per 32-row quarter of the tile (warps q, q + 4, ... share the
//               tensor-memory lanes of quarter q and take every kEpiSub-th 32-column chunk: one
//               epilogue warp per scheduler is bound by its own instruction latencies, two
//               interleave): tcgen05.ld the fp32 accumulator, add bias/residual,
//               convert and store; runs while the next tile's mainloop fills the
//               other accumulator buffer (two TMEM buffers of BN columns).  Nothing
//               the epilogue needs from global memory is fetched on its critical
//               path: the tile's bias row (and, with a folded LayerNorm, the weight
//               column sums and the row's mean / rstd) is staged while the MMAs still
//               run, the residual of a warp's next chunk is fetched during its current
//               one, and a thread stores its 64 bytes of a chunk as two whole sectors.
//               One accumulator chunk is loaded at a time: more loads in flight per
//               warp measured slower, a second warp per scheduler faster.
//
// Tile width BN (32..256), an optional K split and CTA pairing are chosen per
// problem by the host.  With a K split of S, the S CTAs of a thread-block cluster
// each run 1/S of the K loop of the same tile and reduce through distributed shared
// memory: every CTA owns BN/S output columns, receives the peers' fp32 partial sums
// for them by remote shared-memory stores, adds its own accumulator and stores.  This
// keeps all SMs busy when a strip's problem has only a handful of tiles.  With
// pairing, two CTAs form one 256-row tile (cta_group::2): each stages its own 128
// rows of A and half of the B tile, every copy reports its bytes to the even CTA's
// "full" barrier, and the even CTA issues the MMAs and frees the stage in both.
//
// With static weights (bxl_set_static_weights) the B producer does not wait for the
// preceding kernel: weight tiles arrive while that kernel drains.
//
// Roofline: tensor cores.  Algorithmic FLOPs per tile = 2*128*BN*K.
#include <math.h>

#include "bxl_common.cuh"
#include "bxl_host.h"
#include "../../include/basedxl_b200.h"

namespace bxl {

constexpr int kBM = 128;           // tile rows (= TMEM lanes, UMMA M)
constexpr int kBK = 64;            // K per stage: 64 fp16 = one 128-byte swizzle row
constexpr int kUmmaK = 16;         // K of one tcgen05.mma.kind::f16
#ifndef BXL_EPI_SUB
#define BXL_EPI_SUB 2
#endif
constexpr int kEpiSub = BXL_EPI_SUB;            // epilogue warps per 32-row quarter of the tile
constexpr int kEpiThreads = kEpiSub * 128;
constexpr int kWarpA = 4 * kEpiSub, kWarpMma = kWarpA + 1, kWarpB = kWarpA + 2;   // after the epilogue warps: A loads, MMA, B loads
constexpr int kGemmThreads = (4 * kEpiSub + 3) * 32;
constexpr int kMaxSeg = 3;
constexpr int kABytes = kBM * kBK * 2;       // 16 KB
constexpr int kSmemBudget = 227 * 1024;      // dynamic shared memory available to one CTA
constexpr int kSmemMisc = 3072;              // alignment slack + barriers + the tile's bias row (256 floats)
constexpr int kMaxStages = 8;

struct alignas(64) GemmParams {
  CUtensorMap a_map[kMaxSeg];  // GEMM: A of each segment.  conv: body (one row per copy), top halo, bottom halo
  CUtensorMap b_map[kMaxSeg];  // GEMM: B of each segment.  conv: [0] = packed weights
  CUtensorMap a_rows_map;      // conv: body again, with a box of `th` rows (one copy per stage)
  // problem
  int M, N, K;                 // conv: M = B*H_out*W_out (unused), N = C_out, K = 9*C_in
  int nseg;                    // GEMM segments (1, or 3 for the split-operand product)
  int b_kn;                    // B given as [K,N] row-major (MN-major operand) instead of [N,K]
  // tiling chosen by the host
  int bn;                      // tile width: multiple of 32, 32..256
  int split;                   // K split over a cluster of `split` CTAs (1, 2 or 4)
  int pair;                    // CTA pairs (cta_group::2): 256-row tiles, each CTA stages half of B (split == 1)
  int stages;                  // depth of the operand ring
  int b_static;                // B (weights) is not written by the preceding kernel: its copies start before the grid dependency wait
  int n_fastest;               // tile order: 0 = consecutive tiles walk M (they share a B tile), 1 = they walk N (they share an A tile)
  // epilogue
  const __half* bias;          // [N] or null
  const __half* bias_rows;     // conv only: [B][N] per-image bias (time embedding) or null
  long long ld_bias_rows;      // row stride of bias_rows in elements
  const __half* residual;      // [M][ldr] or null
  long long ldr;
  void* C;
  long long ldc;
  int out_f32;
  // optional second destination: output columns >= n_split go to C2[:, col - n_split] (row stride ldc2);
  // n_split is a multiple of 32 (0 = single destination).  Used to write q and k|v of one fused projection
  // to different buffers (the K/V staging slot has its own row stride).
  void* C2;
  long long ldc2;
  int n_split;
  int geglu;                   // epilogue pairs columns: out[16c+i] = h[32c+i] * gelu(h[32c+16+i]), N_out = N/2
  // LayerNorm folded into this GEMM: A holds the UN-normalised rows and B the weights scaled by the
  // LayerNorm gain; with mean_m / rstd_m of row m (from the partial sums its producer wrote) the
  // epilogue forms rstd_m * (acc[m,n] - mean_m * colsum[n]) before bias and the rest.
  const float2* ln_part;       // [M][ln_parts] partial (sum, sum of squares) of every row of A, or null
  int ln_parts;
  float ln_inv_k, ln_eps;      // 1 / row length, epsilon
  const float* ln_colsum;      // [N]: sum over k of B[n,k]
  const float* bias_f32;       // [N] fp32 bias, used instead of `bias` when set
  // Row statistics of the fp16 output (for a LayerNorm folded into the NEXT GEMM): one partial
  // (sum, sum of squares) per row and per column slice a CTA owns, [M][stat_parts].
  float2* stat_out;
  int stat_parts;
  // conv geometry
  int cB, cHin, cW, cCin, cStride, cHout, cWout;
  int tw, th;                  // tile = th rows x tw columns of output pixels (th*tw = 128)
  int tiles_x, tiles_y;        // tiles per image
  int has_top, has_bot;
  int* dev_status;
};

// Split-K exchange buffer of one CTA: for each of the (split-1) peers, the fp32
// partial sums of this CTA's column slice, stored [16-byte chunk][row] so that the
// 32 rows a warp writes (or reads) at once are contiguous.
__host__ __device__ inline int recv_bytes(int bn, int split) { return split > 1 ? (split - 1) * (bn / split) * kBM * 4 : 0; }

// Bias, per-image bias, residual, conversion and the global store of 32 consecutive
// output columns [nb, nb+32) of one output row.
// Residual values of one full-width chunk (32 halves of this thread's output row), fetched a
// chunk ahead of their use.
struct ResidualChunk {
  uint4 u[4];
  bool valid;
};
__device__ __forceinline__ void load_residual(const GemmParams& p, long long out_row, int nb, ResidualChunk& r) {
  r.valid = (p.residual != nullptr) && out_row >= 0 && (nb + 32 <= p.N);
  if (r.valid) {
    const __half* rr = p.residual + out_row * p.ldr + nb;
#pragma unroll
    for (int q = 0; q < 4; ++q) r.u[q] = *reinterpret_cast<const uint4*>(rr + q * 8);
  }
}

// `sbias` = the tile's bias row in shared memory (bias + per-image bias, zero beyond N), indexed
// from the tile's first column; `res` = this chunk's residual if it was prefetched.
// LayerNorm fold of one row: out = ln.a * acc + ln.b * colsum (a = rstd, b = -rstd * mean)
struct LnRow {
  float a, b;
};
// running (sum, sum of squares) of the fp16 values a thread has stored for its row
struct RowStat {
  float s, q;
};

template <bool kConv>
__device__ __forceinline__ void store_chunk(const GemmParams& p, float (&f)[32], long long out_row, int nb, int img,
                                            const float* sbias, const ResidualChunk& res, const float* scol, const LnRow& ln,
                                            RowStat& st) {
  const bool fullw = (nb + 32 <= p.N);
  if (!kConv && scol) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float4 c4 = *reinterpret_cast<const float4*>(scol + 4 * q);
      f[4 * q] = fmaf(ln.a, f[4 * q], ln.b * c4.x), f[4 * q + 1] = fmaf(ln.a, f[4 * q + 1], ln.b * c4.y);
      f[4 * q + 2] = fmaf(ln.a, f[4 * q + 2], ln.b * c4.z), f[4 * q + 3] = fmaf(ln.a, f[4 * q + 3], ln.b * c4.w);
    }
  }
  if (sbias) {
#pragma unroll
    for (int q = 0; q < 8; ++q) {
      const float4 b4 = *reinterpret_cast<const float4*>(sbias + 4 * q);
      f[4 * q] += b4.x, f[4 * q + 1] += b4.y, f[4 * q + 2] += b4.z, f[4 * q + 3] += b4.w;
    }
  }
  if (!kConv && p.geglu) {
    // columns arrive interleaved in groups of 16 values + 16 gates (weight rows were permuted by the
    // caller); N is a multiple of 32 here, so the chunk is always complete
    __half* cr = static_cast<__half*>(p.C) + out_row * p.ldc + (nb >> 1);
    uint32_t w[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int i = 2 * j;
      const float g0 = f[16 + i], g1 = f[16 + i + 1];
      const float y0 = f[i] * (0.5f * g0 * (1.f + erff(g0 * 0.70710678118654752f)));
      const float y1 = f[i + 1] * (0.5f * g1 * (1.f + erff(g1 * 0.70710678118654752f)));
      const __half2 h = __floats2half2_rn(y0, y1);
      w[j] = *reinterpret_cast<const uint32_t*>(&h);
    }
    if ((reinterpret_cast<uintptr_t>(cr) & 31u) == 0) {
      st_global_v8(cr, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);  // the thread's 32 bytes: one whole sector
    } else {
      *reinterpret_cast<uint4*>(cr) = make_uint4(w[0], w[1], w[2], w[3]);
      *reinterpret_cast<uint4*>(cr + 8) = make_uint4(w[4], w[5], w[6], w[7]);
    }
    return;
  }
  if (p.residual) {
    const __half* rr = p.residual + out_row * p.ldr + nb;
    if (fullw) {
#pragma unroll
      for (int q = 0; q < 4; ++q) {
        const uint4 u = res.valid ? res.u[q] : *reinterpret_cast<const uint4*>(rr + q * 8);
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 g = __half22float2(h[j]);
          f[q * 8 + 2 * j] += g.x;
          f[q * 8 + 2 * j + 1] += g.y;
        }
      }
    } else {
      for (int j = 0; j < 32; ++j)
        if (nb + j < p.N) f[j] += __half2float(rr[j]);
    }
  }
  if (p.out_f32) {
    float* cr = static_cast<float*>(p.C) + out_row * p.ldc + nb;
    if (fullw) {
#pragma unroll
      for (int q = 0; q < 8; ++q)
        *reinterpret_cast<float4*>(cr + q * 4) = make_float4(f[q * 4], f[q * 4 + 1], f[q * 4 + 2], f[q * 4 + 3]);
    } else {
      for (int j = 0; j < 32; ++j)
        if (nb + j < p.N) cr[j] = f[j];
    }
  } else {
    __half* cr = (!kConv && p.n_split && nb >= p.n_split)
                     ? static_cast<__half*>(p.C2) + out_row * p.ldc2 + (nb - p.n_split)
                     : static_cast<__half*>(p.C) + out_row * p.ldc + nb;
    if (fullw) {
      uint32_t w[16];
#pragma unroll
      for (int j = 0; j < 16; ++j) {
        const __half2 h = __floats2half2_rn(f[2 * j], f[2 * j + 1]);
        w[j] = *reinterpret_cast<const uint32_t*>(&h);
      }
      if (!kConv && p.stat_out) {
        // statistics of the values as stored (rounded to fp16): what the next GEMM will read
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const float2 g = __half22float2(*reinterpret_cast<const __half2*>(&w[j]));
          st.s += g.x + g.y;
          st.q = fmaf(g.x, g.x, fmaf(g.y, g.y, st.q));
        }
      }
      if ((reinterpret_cast<uintptr_t>(cr) & 31u) == 0) {
        // whole 32-byte sectors: a thread owns 64 contiguous bytes of its row
        st_global_v8(cr, w[0], w[1], w[2], w[3], w[4], w[5], w[6], w[7]);
        st_global_v8(cr + 16, w[8], w[9], w[10], w[11], w[12], w[13], w[14], w[15]);
      } else {
#pragma unroll
        for (int q = 0; q < 4; ++q) *reinterpret_cast<uint4*>(cr + q * 8) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
      }
    } else {
      for (int j = 0; j < 32; ++j)
        if (nb + j < p.N) cr[j] = __float2half_rn(f[j]);
    }
  }
}

// kSplit: the K loop is split over the CTAs of a cluster (p.split of them); a separate
// instantiation, so that each variant carries only its own epilogue (and its registers).
template <bool kConv, bool kPair, bool kSplit>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_conv_kernel(const __grid_constant__ GemmParams p) {
  static_assert(!(kPair && kSplit), "a CTA pair walks the whole K range");
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const int BN = p.bn;
  const int S = kSplit ? p.split : 1;
  const int b_rows = kPair ? BN / 2 : BN;       // rows of the B tile this CTA stages
  const int stage_bytes = kABytes + b_rows * 128;
  constexpr int kWidth = kPair ? 2 : 1;          // CTAs that cooperate on one tile (besides a K split)
  const uint32_t recv_base = smem_base + p.stages * stage_bytes;            // 1024-aligned (stage_bytes % 1024 == 0)
  const uint32_t bar_base = recv_base + recv_bytes(BN, S);
  // barriers (8 bytes each): full[kMaxStages], empty[kMaxStages], tfull[2], tempty[2], recv_full, recv_free
  auto full_bar = [&](int s) { return bar_base + 8u * s; };
  auto empty_bar = [&](int s) { return bar_base + 8u * (kMaxStages + s); };
  auto tfull_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + a); };
  auto tempty_bar = [&](int a) { return bar_base + 8u * (2 * kMaxStages + 2 + a); };
  const uint32_t recv_full_bar = bar_base + 8u * (2 * kMaxStages + 4);
  const uint32_t recv_free_bar = bar_base + 8u * (2 * kMaxStages + 5);
  uint8_t* misc = smem_gen + (bar_base - smem_base) + 256;
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(misc);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(misc + 8);
  float* s_bias = reinterpret_cast<float*>(misc + 256);   // [256]: bias row of the tile in the epilogue
  float* s_colsum = s_bias + 256;                         // [256]: weight column sums (LayerNorm fold only; the host sizes the CTA for it)

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t tmem_cols = (2 * BN <= 64) ? 64u : (2 * BN <= 128) ? 128u : (2 * BN <= 256) ? 256u : 512u;
  const uint32_t crank = (S > 1 || kPair) ? cluster_ctarank() : 0u;

  if (threadIdx.x == 0) {
    for (int s = 0; s < p.stages; ++s) {
      // one arrival (with its byte count) from each of this CTA's two producer threads
      mbar_init(full_bar(s), 2);
      mbar_init(empty_bar(s), 1);
    }
    for (int a = 0; a < 2; ++a) {
      mbar_init(tfull_bar(a), 1);
      mbar_init(tempty_bar(a), 4 * kEpiSub * kWidth);  // one arrival per epilogue warp (of both CTAs in pair mode)
    }
    const uint32_t peers_threads = (S > 1) ? (S - 1) * static_cast<uint32_t>(kEpiThreads) : 1u;  // every epilogue thread of every peer
    mbar_init(recv_full_bar, peers_threads);
    mbar_init(recv_free_bar, peers_threads);
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == kWarpMma) {
    if (kPair) {
      tmem_alloc_pair(smem_u32(const_cast<uint32_t*>(tmem_slot)), tmem_cols);
      tmem_relinquish_pair();
    } else {
      tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), tmem_cols);
      tmem_relinquish();
    }
  }
  tc_fence_before_sync();
  __syncthreads();
  if (S > 1 || kPair) cluster_sync_all();  // peers' barriers are initialised before anyone arrives on them
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // Everything above overlaps the previous kernel's tail; global data from here on.  With static
  // weights the B producer does not wait: it fills the ring with B tiles while the previous
  // kernel finishes (A, written by that kernel, is only loaded after the wait).
  if (!(p.b_static && warp == kWarpB)) pdl_wait();

  // ---- tile enumeration ------------------------------------------------------
  const int tiles_n = (p.N + BN - 1) / BN;
  int tiles_m1;  // 128-row tiles
  if (kConv) tiles_m1 = p.cB * p.tiles_y * p.tiles_x;
  else tiles_m1 = (p.M + kBM - 1) / kBM;
  const int tiles_m = kPair ? (tiles_m1 + 1) / 2 : tiles_m1;  // scheduling units along M (pairs of tiles in pair mode)
  const int num_tiles = tiles_m * tiles_n;
  const int kb_per_seg = kConv ? 9 * (p.cCin / kBK) : (p.K + kBK - 1) / kBK;
  const int num_kb = kConv ? kb_per_seg : kb_per_seg * p.nseg;
  // this CTA's share of the K loop (balanced; never empty because split <= num_kb)
  const uint32_t krank = kPair ? 0u : crank;  // both CTAs of a pair walk the whole K range
  const int kb_begin = static_cast<int>((static_cast<long long>(krank) * num_kb) / S);
  const int kb_end = static_cast<int>((static_cast<long long>(krank + 1) * num_kb) / S);
  const int first_tile = blockIdx.x / (S * kWidth);
  const int tile_step = gridDim.x / (S * kWidth);

  if (warp == kWarpA || warp == kWarpB) {
    // ======================= TMA producers =======================
    // Issuing a tiled copy occupies the issuing thread for a few hundred cycles, so the A
    // and B operands are fed by two threads in different warps; both arrive on the stage's
    // "full" barrier with the bytes they ordered.
    const bool loads_a = (warp == kWarpA);
    if (lane == 0) {
      for (int s = 0; s < kMaxSeg; ++s) tma_prefetch_desc(loads_a ? &p.a_map[s] : &p.b_map[s]);
      if (loads_a && kConv) tma_prefetch_desc(&p.a_rows_map);
      int stage = 0;
      uint32_t phase = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step) {
        const int tm = (p.n_fastest ? tile / tiles_n : tile % tiles_m) * kWidth + (kPair ? static_cast<int>(crank) : 0);  // this CTA's 128-row tile
        const int tn = p.n_fastest ? tile % tiles_n : tile / tiles_m;
        const int n0 = tn * BN + (kPair ? static_cast<int>(crank) * b_rows : 0);           // first B row this CTA stages
        int img = 0, y0 = 0, x0 = 0;
        if (kConv) {
          // a pair's second tile may lie past the last image: its copies are then entirely out of
          // bounds (zero fill) and its rows are not stored
          const int per_img = p.tiles_y * p.tiles_x;
          img = tm / per_img;
          const int r = tm % per_img;
          y0 = (r / p.tiles_x) * p.th;
          x0 = (r % p.tiles_x) * p.tw;
        }
        // position in the K loop, advanced without divisions: this thread's issue rate bounds the
        // pipeline ramp of short K loops
        const int cchunks = kConv ? p.cCin / kBK : 1;
        int seg = kConv ? 0 : kb_begin / kb_per_seg;        // GEMM: operand segment and k-block inside it
        int kk = kConv ? 0 : kb_begin % kb_per_seg;
        int tap = kConv ? kb_begin / cchunks : 0;           // conv: filter tap (ky, kx) and channel chunk
        int cc = kConv ? kb_begin % cchunks : 0;
        int ky = tap / 3, kx = tap % 3;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (!mbar_wait(empty_bar(stage), phase ^ 1u, abort_flag, p.dev_status, loads_a ? 100 : 101)) {
            ok = false;
            break;
          }
          const uint32_t a_dst = smem_base + stage * stage_bytes;
          const uint32_t b_dst = a_dst + kABytes;
          // pair mode: both CTAs report their bytes to the leader's barrier; the leader's two
          // producer threads announce the bytes of both halves
          const uint32_t fbar = kPair ? map_to_cta(full_bar(stage), 0) : full_bar(stage);
          const bool announces = !kPair || crank == 0;
          auto load_2d = [&](uint32_t dst, const CUtensorMap* m, int c0, int c1) {
            if (kPair) tma_load_2d_pair(dst, m, fbar, c0, c1);
            else tma_load_2d(dst, m, fbar, c0, c1);
          };
          auto load_5d = [&](uint32_t dst, const CUtensorMap* m, int c0, int c1, int c2, int c3, int c4) {
            if (kPair) tma_load_5d_pair(dst, m, fbar, c0, c1, c2, c3, c4);
            else tma_load_5d(dst, m, fbar, c0, c1, c2, c3, c4);
          };
          if (loads_a) {
            if (announces) mbar_arrive_expect_tx(full_bar(stage), kABytes * kWidth);
            if (kConv) {
              const int c0 = cc * kBK;
              // input column of output column ox: stride*ox + kx - 1, addressed as
              // (parity, half-column) = ((kx-1) mod stride, ox + floor((kx-1)/stride))
              int par = 0, xoff = kx - 1;
              if (p.cStride == 2) {
                par = (kx == 1) ? 0 : 1;
                xoff = (kx == 0) ? -1 : 0;
              }
              const int r_first = p.cStride * y0 + ky - 1;
              const int r_last = p.cStride * (y0 + p.th - 1) + ky - 1;
              const bool touches_halo = (p.has_top && r_first < 0) || (p.has_bot && r_last >= p.cHin);
              if (p.cStride == 1 && !touches_halo) {
                // all th input rows come from the body (rows outside [0, H) are zero-filled by
                // the copy engine): one copy for the whole A tile
                load_5d(a_dst, &p.a_rows_map, c0, par, x0 + xoff, r_first, img);
              } else {
                for (int t = 0; t < p.th; ++t) {
                  const int r_in = p.cStride * (y0 + t) + ky - 1;
                  const uint32_t dst = a_dst + t * p.tw * 128;
                  const CUtensorMap* src = (r_in == -1 && p.has_top) ? &p.a_map[1] : (r_in == p.cHin && p.has_bot) ? &p.a_map[2] : &p.a_map[0];
                  const int r_src = (src == &p.a_map[0]) ? r_in : 0;
                  load_5d(dst, src, c0, par, x0 + xoff, r_src, img);
                }
              }
            } else {
              load_2d(a_dst, &p.a_map[seg], kk * kBK, tm * kBM);
            }
          } else {
            if (announces) mbar_arrive_expect_tx(full_bar(stage), b_rows * 128 * kWidth);
            if (kConv) {
              load_2d(b_dst, &p.b_map[0], kb * kBK, n0);
            } else {
              const int k0 = kk * kBK;
              if (p.b_kn) {
                // B[K,N]: one 64(n) x 64(k) box per 64 output columns
                for (int j = 0; j < b_rows / 64; ++j) load_2d(b_dst + j * 8192, &p.b_map[seg], n0 + j * 64, k0);
              } else {
                load_2d(b_dst, &p.b_map[seg], k0, n0);
              }
            }
          }
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
          if (kConv) {
            if (++cc == cchunks) {
              cc = 0;
              if (++kx == 3) kx = 0, ++ky;
            }
          } else if (++kk == kb_per_seg) {
            kk = 0, ++seg;
          }
        }
      }
    }
  } else if (warp == kWarpMma) {
    // ======================= MMA issuer =======================
    if (kPair && crank != 0) {
      // odd CTA of a pair: the leader issues the MMAs for both
    } else if (lane == 0) {
      const uint32_t idesc = make_idesc_f16(kBM * kWidth, BN, 0, (!kConv && p.b_kn) ? 1 : 0);
      int stage = 0;
      uint32_t phase = 0;
      int it = 0;
      bool ok = true;
      for (int tile = first_tile; tile < num_tiles && ok; tile += tile_step, ++it) {
        const int acc = it & 1;
        const uint32_t acc_phase = (it >> 1) & 1u;
        if (kPair ? !mbar_wait_cluster(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.dev_status, 200)
                  : !mbar_wait(tempty_bar(acc), acc_phase ^ 1u, abort_flag, p.dev_status, 200))
          break;
        tc_fence_after_sync();
        const uint32_t d_tmem = tmem_base + acc * BN;
        for (int kb = kb_begin; kb < kb_end; ++kb) {
          if (kPair ? !mbar_wait_cluster(full_bar(stage), phase, abort_flag, p.dev_status, 201)
                    : !mbar_wait(full_bar(stage), phase, abort_flag, p.dev_status, 201)) {
            ok = false;
            break;
          }
          tc_fence_after_sync();
          const uint32_t a_addr = smem_base + stage * stage_bytes;
          const uint32_t b_addr = a_addr + kABytes;
          const uint64_t adesc = make_smem_desc_sw128(a_addr, 16, 1024);
          const uint32_t first = (kb == kb_begin) ? 0u : 1u;
          if (!kConv && p.b_kn) {
            // MN-major B: 64-column chunks 8 KB apart (LBO), 8-row k-groups 1 KB apart (SBO)
            const uint64_t bdesc = make_smem_desc_sw128(b_addr, 8192, 1024);
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k) {
              if (kPair) umma_f16_pair(d_tmem, adesc + 2u * k, bdesc + 128u * k, idesc, first | k);
              else umma_f16(d_tmem, adesc + 2u * k, bdesc + 128u * k, idesc, first | k);
            }
          } else {
            const uint64_t bdesc = make_smem_desc_sw128(b_addr, 16, 1024);
#pragma unroll
            for (int k = 0; k < kBK / kUmmaK; ++k) {
              if (kPair) umma_f16_pair(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, first | k);
              else umma_f16(d_tmem, adesc + 2u * k, bdesc + 2u * k, idesc, first | k);
            }
          }
          // frees the stage (in both CTAs of a pair) once these MMAs have read it
          if (kPair) {
            umma_commit_pair(empty_bar(stage));
            umma_commit_pair(map_to_cta(empty_bar(stage), 1));
          } else {
            umma_commit(empty_bar(stage));
          }
          if (++stage == p.stages) {
            stage = 0;
            phase ^= 1u;
          }
        }
        if (ok) {
          if (kPair) {
            umma_commit_pair(tfull_bar(acc));
            umma_commit_pair(map_to_cta(tfull_bar(acc), 1));
          } else {
            umma_commit(tfull_bar(acc));
          }
        }
      }
    }
  } else {
    // ======================= epilogue (warps 0..7) =======================
    const int quarter = warp & 3;  // TMEM lane quarter this warp may access
    const int half = warp >> 2;    // which of the quarter's kEpiSub warps: it takes the chunks c with c % kEpiSub == half
    const int row_in_tile = quarter * 32 + lane;
    const int chunks = BN / 32;
    const int cps = chunks / S;    // 32-column chunks per owner slice
    int it = 0;
    for (int tile = first_tile; tile < num_tiles; tile += tile_step, ++it) {
      const int acc = it & 1;
      const uint32_t acc_phase = (it >> 1) & 1u;
      const int tm = (p.n_fastest ? tile / tiles_n : tile % tiles_m) * kWidth + (kPair ? static_cast<int>(crank) : 0);
      const int tn = p.n_fastest ? tile % tiles_n : tile / tiles_m;
      const int n0 = tn * BN;
      long long out_row = -1;  // row index into C / residual, -1 = not stored
      int img = 0;
      if (kConv) {
        const int per_img = p.tiles_y * p.tiles_x;
        img = tm / per_img;
        const int r = tm % per_img;
        const int oy = (r / p.tiles_x) * p.th + row_in_tile / p.tw;
        const int ox = (r % p.tiles_x) * p.tw + row_in_tile % p.tw;
        if (img < p.cB && oy < p.cHout && ox < p.cWout) out_row = (static_cast<long long>(img) * p.cHout + oy) * p.cWout + ox;
      } else {
        const int m = tm * kBM + row_in_tile;
        if (m < p.M) out_row = m;
      }
      // Stage the tile's bias row while the MMAs of this tile are still running.  The four
      // epilogue warps meet on named barrier 1 twice: nobody still reads the previous tile's
      // row when it is overwritten, and the new row is complete before anybody reads it.
      const bool has_ln = !kConv && (p.ln_part != nullptr);
      const bool has_bias = (p.bias != nullptr) || (p.bias_f32 != nullptr) || (kConv && p.bias_rows != nullptr);
      if (has_bias || has_ln) {
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
        const int et = warp * 32 + lane;   // 0..kEpiThreads-1
        for (int j = et; j < BN; j += kEpiThreads) {
          float b = 0.f, cs = 0.f;
          if (n0 + j < p.N) {
            if (p.bias_f32) b += p.bias_f32[n0 + j];
            else if (p.bias) b += __half2float(p.bias[n0 + j]);
            if (kConv && p.bias_rows && img < p.cB) b += __half2float(p.bias_rows[static_cast<long long>(img) * p.ld_bias_rows + n0 + j]);
            if (has_ln) cs = p.ln_colsum[n0 + j];
          }
          s_bias[j] = b;
          if (has_ln) s_colsum[j] = cs;
        }
        asm volatile("bar.sync 1, %0;" ::"n"(kEpiThreads) : "memory");
      }
      // LayerNorm fold: this row's mean and reciprocal standard deviation from the partial sums
      // the producer of A left (read while this tile's MMAs still run)
      LnRow ln{1.f, 0.f};
      if (has_ln && out_row >= 0) {
        const float2* pp = p.ln_part + out_row * p.ln_parts;
        float sm = 0.f, sq = 0.f;
        for (int i = 0; i < p.ln_parts; ++i) {
          const float2 v = pp[i];
          sm += v.x, sq += v.y;
        }
        const float mean = sm * p.ln_inv_k;
        const float var = fmaxf(sq * p.ln_inv_k - mean * mean, 0.f);
        ln.a = rsqrtf(var + p.ln_eps);
        ln.b = -ln.a * mean;
      }
      RowStat stat{0.f, 0.f};
      // This warp's chunks are c = half, half + 2, ... ; the residual of a chunk is fetched while
      // the chunk before it (of this warp) is converted and stored.
      ResidualChunk res_cur, res_next;
      res_cur.valid = res_next.valid = false;
      if (!kSplit) {
        // the residual of the first chunk travels while the MMAs of this tile still run
        if (half < chunks) load_residual(p, out_row, n0 + half * 32, res_cur);
      }
      if (!mbar_wait(tfull_bar(acc), acc_phase, abort_flag, p.dev_status, 300)) break;
      __syncwarp();
      tc_fence_after_sync();
      const uint32_t t_row = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16) + acc * BN;
      if constexpr (!kSplit) {
        // One chunk at a time per warp (measured: several accumulator loads in flight per warp do not
        // shorten the epilogue; a second warp on the same scheduler does).
#pragma unroll 1
        for (int c = half; c < chunks; c += kEpiSub) {
          uint32_t v[32];
          tmem_ld_32x32(t_row + c * 32, v);
          if (c + kEpiSub < chunks) load_residual(p, out_row, n0 + (c + kEpiSub) * 32, res_next);
          tmem_ld_wait();
          const int nb = n0 + c * 32;
          if (out_row >= 0 && nb < p.N) {
            float f[32];
#pragma unroll
            for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
            store_chunk<kConv>(p, f, out_row, nb, img, has_bias ? s_bias + c * 32 : nullptr, res_cur,
                               has_ln ? s_colsum + c * 32 : nullptr, ln, stat);
          }
          res_cur = res_next;
          res_next.valid = false;
        }
      } else {
        // ---- split-K: push the partial sums of the peers' column slices into their
        //      exchange buffers, then reduce and store this CTA's own slice ----
        // peers must have finished reading what was pushed for the previous tile
        if (it > 0 && !mbar_wait_cluster(recv_free_bar, (it - 1) & 1u, abort_flag, p.dev_status, 301)) break;
        __syncwarp();
        {
          const int own_lo = static_cast<int>(crank) * cps;
          const int nf = chunks - cps;                                  // chunks owned by the peers
#pragma unroll 1
          for (int fi = half; fi < nf; fi += kEpiSub) {
            const int c = fi < own_lo ? fi : fi + cps;                   // fi-th chunk that is not this CTA's own
            uint32_t v[32];
            tmem_ld_32x32(t_row + c * 32, v);
            tmem_ld_wait();
            const uint32_t owner = c / cps;
            const uint32_t slot = (crank < owner) ? crank : crank - 1;   // this CTA's slot at the owner
            const uint32_t base = recv_base + ((slot * cps + (c % cps)) * 8u * kBM + row_in_tile) * 16u;
            const uint32_t remote = map_to_cta(base, owner);
#pragma unroll
            for (int q = 0; q < 8; ++q)
              st_cluster_f32x4(remote + q * kBM * 16u, __uint_as_float(v[4 * q]), __uint_as_float(v[4 * q + 1]),
                               __uint_as_float(v[4 * q + 2]), __uint_as_float(v[4 * q + 3]));
          }
        }
        for (uint32_t o = 0; o < static_cast<uint32_t>(S); ++o)
          if (o != crank) mbar_arrive_remote(map_to_cta(recv_full_bar, o));
        // own slice (this warp's chunks of it): wait for every peer's partials; the first chunk's
        // residual and accumulator load travel meanwhile
        const bool has_own = half < cps;
        uint32_t v[32];
        if (has_own) {
          load_residual(p, out_row, n0 + (static_cast<int>(crank) * cps + half) * 32, res_cur);
          tmem_ld_32x32(t_row + (static_cast<int>(crank) * cps + half) * 32, v);
        }
        if (!mbar_wait_cluster(recv_full_bar, it & 1u, abort_flag, p.dev_status, 302)) break;
        __syncwarp();
#pragma unroll 1
        for (int cc = half; cc < cps; cc += kEpiSub) {
          const int c = crank * cps + cc;
          if (cc + kEpiSub < cps) load_residual(p, out_row, n0 + (c + kEpiSub) * 32, res_next);
          tmem_ld_wait();
          float f[32];
#pragma unroll
          for (int j = 0; j < 32; ++j) f[j] = __uint_as_float(v[j]);
          if (cc + kEpiSub < cps) tmem_ld_32x32(t_row + (c + kEpiSub) * 32, v);   // this warp's next own chunk, in flight during the reduction
          for (int slot = 0; slot < S - 1; ++slot) {
            const uint8_t* src = smem_gen + (recv_base - smem_base) + ((slot * cps + cc) * 8 * kBM + row_in_tile) * 16;
#pragma unroll
            for (int q = 0; q < 8; ++q) {
              const float4 g = *reinterpret_cast<const float4*>(src + q * kBM * 16);
              f[4 * q] += g.x, f[4 * q + 1] += g.y, f[4 * q + 2] += g.z, f[4 * q + 3] += g.w;
            }
          }
          const int nb = n0 + c * 32;
          if (out_row >= 0 && nb < p.N)
            store_chunk<kConv>(p, f, out_row, nb, img, has_bias ? s_bias + c * 32 : nullptr, res_cur,
                               has_ln ? s_colsum + c * 32 : nullptr, ln, stat);
          res_cur = res_next;
          res_next.valid = false;
        }
        // tell the peers their pushes have been consumed
        for (uint32_t o = 0; o < static_cast<uint32_t>(S); ++o)
          if (o != crank) mbar_arrive_remote(map_to_cta(recv_free_bar, o));
      }
      if (!kConv && p.stat_out && out_row >= 0)
        p.stat_out[out_row * p.stat_parts + (tn * S + (S > 1 ? static_cast<int>(crank) : 0)) * kEpiSub + half] = make_float2(stat.s, stat.q);
      tc_fence_before_sync();
      __syncwarp();
      if (lane == 0) {
        if (kPair && crank != 0) mbar_arrive_remote(map_to_cta(tempty_bar(acc), 0));
        else mbar_arrive(tempty_bar(acc));
      }
    }
  }

  // ---- teardown ---------------------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    // give copies that may still be in flight time to land before the CTA's
    // shared memory is released
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  // no CTA of a cluster may leave while a peer can still write into its shared memory
  if (S > 1 || kPair) cluster_sync_all();
  if (warp == kWarpMma) {
    __syncwarp();
    tc_fence_after_sync();
    if (kPair) tmem_dealloc_pair(tmem_base, tmem_cols);
    else tmem_dealloc(tmem_base, tmem_cols);
  }
}

// ---------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------
struct TileConfig {
  int bn, split, stages, pair;
};

constexpr int kSmemLnExtra = 1024;           // the weight column-sum row of a GEMM with a folded LayerNorm

static int stages_for(int bn, int split, int pair = 0, int extra_smem = 0) {
  const int stage = kABytes + (pair ? bn * 64 : bn * 128);
  int st = (kSmemBudget - kSmemMisc - extra_smem - recv_bytes(bn, split)) / stage;
  if (st > kMaxStages) st = kMaxStages;
  return st;
}

// Pick the tile width, the K split and whether to pair CTAs, minimising a time model fitted
// to a sweep of every (tile width, split, pairing) over the GEMM and convolution shapes of the
// SDXL UNet on B200.  One CTA streams its operands at ~110 KB/us from L2 (the per-SM fill rate
// bounds these kernels, not the tensor pipe), so a k-block of a 128 x bn tile costs
// max(mma(bn), bytes / 110 KB/us) with bytes = 16 KB + bn*128 B.  A CTA pair moves half of the B
// tile per CTA but its stage recycling crosses two SMs: 0.24 us + 0.63 ns * bn per k-block.
// `a_min_us` is a floor per k-block for the A operand path (the multi-row image copies of the
// convolution).  A wider tile or a pair moves fewer bytes per FLOP; a narrower tile or a K split
// spreads the stream over more SMs when there are few tiles.
static TileConfig choose_tiles(int tiles_m, int N, int num_kb, bool b_kn, int force_bn = 0, int force_split = 0,
                               int force_pair = -1, double a_min_us = 0.0, int extra_smem = 0) {
  const int sms = sm_count();
  TileConfig best{128, 1, stages_for(128, 1, 0, extra_smem), 0};
  double best_cost = 1e30;
  for (int pair = 0; pair <= 1; ++pair) {
    if (force_pair >= 0 && pair != force_pair) continue;
    for (int bn = 32; bn <= 256; bn += 32) {
      if (b_kn && (pair ? bn % 128 : bn % 64)) continue;  // MN-major B is loaded in 64-column boxes
      if (force_bn && bn != force_bn) continue;
      const int units_m = pair ? (tiles_m + 1) / 2 : tiles_m;
      const int tiles = units_m * ((N + bn - 1) / bn);
      for (int split = 1; split <= (pair ? 1 : 4); split *= 2) {
        if (force_split && split != force_split) continue;
        if ((bn / 32) % split || split > num_kb) continue;
        const int st = stages_for(bn, split, pair, extra_smem);
        if (st < 3) continue;
        const int width = pair ? 2 : split;
        const int clusters = sms / width;
        const int par = tiles < clusters ? tiles : clusters;
        const int rounds = (tiles + par - 1) / par;
        const double bytes = 16384.0 + bn * (pair ? 64.0 : 128.0);
        const double kb_us = fmax(fmax(bn / 256.0 * 0.27, pair ? 0.24 + 0.00063 * bn : bytes / 110000.0), a_min_us);
        const double kb_unit = (num_kb + split - 1) / split;
        const double epi_us = 0.08 * (bn / 32.0) / split + (split > 1 ? 1.2 : 0.0);  // accumulator read-out (+ exchange)
        const double fill_us = 1.0 + (st < 4 ? 0.5 : 0.0) + (pair ? 0.3 : 0.0);       // pipeline ramp per unit
        const double pair_tile_us = pair ? 0.45 : 0.0;  // accumulator hand-over between the two CTAs, per tile
        const double cost = rounds * (kb_unit * kb_us + epi_us + pair_tile_us) + fill_us + 3.0;
        if (cost < best_cost - 1e-9) {
          best_cost = cost;
          best = TileConfig{bn, split, st, pair};
        }
      }
    }
  }
  return best;
}

template <bool kConv, bool kPair, bool kSplit>
static int launch_one(const GemmParams& p, int num_units, cudaStream_t stream) {
  const int b_rows = kPair ? p.bn / 2 : p.bn;
  const int smem = p.stages * (kABytes + b_rows * 128) + recv_bytes(p.bn, kSplit ? p.split : 1) + kSmemMisc +
                   (p.ln_part ? kSmemLnExtra : 0);
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (int rc = check_cuda(cudaFuncSetAttribute(gemm_conv_kernel<kConv, kPair, kSplit>, cudaFuncAttributeMaxDynamicSharedMemorySize, kSmemBudget),
                            "cudaFuncSetAttribute(gemm)"))
      return rc;
    configured[dev] = true;
  }
  const int width = kPair ? 2 : (kSplit ? p.split : 1);
  int clusters = sm_count() / width;
  if (clusters > num_units) clusters = num_units;
  if (clusters < 1) clusters = 1;
  return launch_kernel("gemm_conv_kernel launch", gemm_conv_kernel<kConv, kPair, kSplit>, dim3(clusters * width), dim3(kGemmThreads), smem,
                       stream, width, p);
}

// tiles_m: 128-row tiles along M; tiles_n: tiles along N
template <bool kConv>
static int launch(const GemmParams& p, int tiles_m, int tiles_n, cudaStream_t stream) {
  if (p.pair) return launch_one<kConv, true, false>(p, ((tiles_m + 1) / 2) * tiles_n, stream);
  if (p.split > 1) return launch_one<kConv, false, true>(p, tiles_m * tiles_n, stream);
  return launch_one<kConv, false, false>(p, tiles_m * tiles_n, stream);
}

static int aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// test hook: force the tile width / K split (0 = choose)
constexpr int kDefaultPair = -1;  // -1 = let the cost model decide
constexpr double kConvAMinUs = 0.36;  // per-k-block floor of the convolution's image copies
static int g_force_bn = 0, g_force_split = 0, g_force_pair = -1;
static int g_force_order = -1;  // -1 = choose, 0 = consecutive tiles walk M, 1 = they walk N
// Linear layers: an activation matrix that does not stay in L2 beside the output is walked once
// (the CTAs running at one time take the column tiles of the same rows) as long as the weights do.
static int linear_tile_order(long long M, long long N, long long K, int bn) {
  if (g_force_order >= 0) return g_force_order;
  return (N > bn && 2 * M * K > (48ll << 20) && 2 * N * K < (32ll << 20)) ? 1 : 0;
}

}  // namespace bxl

using namespace bxl;

extern "C" int bxl_gemm_f16(const void* A, long long lda, const void* B, long long ldb, int b_is_kn, const void* bias,
                            const void* residual, long long ldr, void* C, long long ldc, int out_f32, int M, int N, int K,
                            void* stream) {
  if (!A || !B || !C) return fail(kErrInvalidArg, "bxl_gemm_f16: null operand");
  if (M <= 0 || N <= 0 || K <= 0) return fail(kErrInvalidArg, "bxl_gemm_f16: non-positive extent M=%d N=%d K=%d", M, N, K);
  if (lda % 8 || ldb % 8) return fail(kErrInvalidArg, "bxl_gemm_f16: lda/ldb must be multiples of 8 elements");
  if (!aligned16(A) || !aligned16(B) || !aligned16(C) || (residual && !aligned16(residual)))
    return fail(kErrInvalidArg, "bxl_gemm_f16: operands must be 16-byte aligned");
  if (ldc % (out_f32 ? 4 : 8) || (residual && ldr % 8))
    return fail(kErrInvalidArg, "bxl_gemm_f16: ldc/ldr must keep rows 16-byte aligned");
  if (lda < K || (b_is_kn ? ldb < N : ldb < K) || ldc < N) return fail(kErrInvalidArg, "bxl_gemm_f16: leading dimension too small");
  int* st = device_status_ptr();
  if (!st) return fail(kErrCuda, "bxl_gemm_f16: no device status word");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const int tiles_m = (M + kBM - 1) / kBM;
  const TileConfig tc = choose_tiles(tiles_m, N, (K + kBK - 1) / kBK, b_is_kn != 0, g_force_bn, g_force_split, g_force_pair < 0 ? kDefaultPair : g_force_pair);
  const int BN = tc.bn;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {kBK, kBM};
    if (int rc = encode_tmap_f16(&p.a_map[0], A, 2, dims, str, box)) return rc;
  }
  if (b_is_kn) {
    uint64_t dims[2] = {(uint64_t)N, (uint64_t)K};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {64, kBK};
    if (int rc = encode_tmap_f16(&p.b_map[0], B, 2, dims, str, box)) return rc;
  } else {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {kBK, (uint32_t)(tc.pair ? BN / 2 : BN)};
    if (int rc = encode_tmap_f16(&p.b_map[0], B, 2, dims, str, box)) return rc;
  }
  for (int s = 1; s < kMaxSeg; ++s) {
    p.a_map[s] = p.a_map[0];
    p.b_map[s] = p.b_map[0];
  }
  p.M = M, p.N = N, p.K = K, p.nseg = 1, p.b_kn = b_is_kn ? 1 : 0;
  p.bn = tc.bn, p.split = tc.split, p.stages = tc.stages, p.pair = tc.pair, p.b_static = static_weights() ? 1 : 0;
  p.n_fastest = linear_tile_order(M, N, K, tc.bn);
  p.bias = static_cast<const __half*>(bias);
  p.residual = static_cast<const __half*>(residual);
  p.ldr = ldr, p.C = C, p.ldc = ldc, p.out_f32 = out_f32 ? 1 : 0;
  p.dev_status = st;
  return launch<false>(p, tiles_m, (N + BN - 1) / BN, (cudaStream_t)stream);
}

extern "C" int bxl_gemm_dual_f16(const void* A, long long lda, const void* B, long long ldb, const void* bias, void* C1,
                                 long long ldc1, int n1, void* C2, long long ldc2, int M, int N, int K, void* stream) {
  if (!A || !B || !C1 || !C2) return fail(kErrInvalidArg, "bxl_gemm_dual_f16: null operand");
  if (M <= 0 || N <= 0 || K <= 0 || n1 <= 0 || n1 >= N || n1 % 32 || N % 8)
    return fail(kErrInvalidArg, "bxl_gemm_dual_f16: need 0 < n1 < N with n1 a multiple of 32 (n1=%d N=%d)", n1, N);
  if (lda % 8 || ldb % 8 || ldc1 % 8 || ldc2 % 8 || lda < K || ldb < K || ldc1 < n1 || ldc2 < N - n1)
    return fail(kErrInvalidArg, "bxl_gemm_dual_f16: bad leading dimension");
  if (!aligned16(A) || !aligned16(B) || !aligned16(C1) || !aligned16(C2))
    return fail(kErrInvalidArg, "bxl_gemm_dual_f16: operands must be 16-byte aligned");
  int* st = device_status_ptr();
  if (!st) return fail(kErrCuda, "bxl_gemm_dual_f16: no device status word");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const int tiles_m = (M + kBM - 1) / kBM;
  const TileConfig tc = choose_tiles(tiles_m, N, (K + kBK - 1) / kBK, false, g_force_bn, g_force_split, g_force_pair < 0 ? kDefaultPair : g_force_pair);
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {kBK, kBM};
    if (int rc = encode_tmap_f16(&p.a_map[0], A, 2, dims, str, box)) return rc;
  }
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {kBK, (uint32_t)(tc.pair ? tc.bn / 2 : tc.bn)};
    if (int rc = encode_tmap_f16(&p.b_map[0], B, 2, dims, str, box)) return rc;
  }
  for (int s = 1; s < kMaxSeg; ++s) {
    p.a_map[s] = p.a_map[0];
    p.b_map[s] = p.b_map[0];
  }
  p.M = M, p.N = N, p.K = K, p.nseg = 1, p.b_kn = 0;
  p.bn = tc.bn, p.split = tc.split, p.stages = tc.stages, p.pair = tc.pair, p.b_static = static_weights() ? 1 : 0;
  p.n_fastest = linear_tile_order(M, N, K, tc.bn);
  p.bias = static_cast<const __half*>(bias);
  p.C = C1, p.ldc = ldc1, p.C2 = C2, p.ldc2 = ldc2, p.n_split = n1;
  p.dev_status = st;
  return launch<false>(p, tiles_m, (N + tc.bn - 1) / tc.bn, (cudaStream_t)stream);
}

extern "C" int bxl_gemm_geglu_f16(const void* A, long long lda, const void* B, long long ldb, const void* bias, void* C,
                                  long long ldc, int M, int N, int K, void* stream) {
  if (!A || !B || !C) return fail(kErrInvalidArg, "bxl_gemm_geglu_f16: null operand");
  if (M <= 0 || N <= 0 || K <= 0 || N % 32) return fail(kErrInvalidArg, "bxl_gemm_geglu_f16: N=%d must be a positive multiple of 32", N);
  if (lda % 8 || ldb % 8 || ldc % 8 || lda < K || ldb < K || ldc < N / 2)
    return fail(kErrInvalidArg, "bxl_gemm_geglu_f16: bad leading dimension");
  if (!aligned16(A) || !aligned16(B) || !aligned16(C)) return fail(kErrInvalidArg, "bxl_gemm_geglu_f16: operands must be 16-byte aligned");
  int* st = device_status_ptr();
  if (!st) return fail(kErrCuda, "bxl_gemm_geglu_f16: no device status word");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const int tiles_m = (M + kBM - 1) / kBM;
  const TileConfig tc = choose_tiles(tiles_m, N, (K + kBK - 1) / kBK, false, g_force_bn, g_force_split, g_force_pair < 0 ? kDefaultPair : g_force_pair);
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)lda * 2};
    uint32_t box[2] = {kBK, kBM};
    if (int rc = encode_tmap_f16(&p.a_map[0], A, 2, dims, str, box)) return rc;
  }
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t str[1] = {(uint64_t)ldb * 2};
    uint32_t box[2] = {kBK, (uint32_t)(tc.pair ? tc.bn / 2 : tc.bn)};
    if (int rc = encode_tmap_f16(&p.b_map[0], B, 2, dims, str, box)) return rc;
  }
  for (int s = 1; s < kMaxSeg; ++s) {
    p.a_map[s] = p.a_map[0];
    p.b_map[s] = p.b_map[0];
  }
  p.M = M, p.N = N, p.K = K, p.nseg = 1, p.b_kn = 0;
  p.bn = tc.bn, p.split = tc.split, p.stages = tc.stages, p.pair = tc.pair, p.b_static = static_weights() ? 1 : 0;
  p.n_fastest = linear_tile_order(M, N, K, tc.bn);
  p.bias = static_cast<const __half*>(bias);
  p.C = C, p.ldc = ldc, p.out_f32 = 0, p.geglu = 1;
  p.dev_status = st;
  return launch<false>(p, tiles_m, (N + tc.bn - 1) / tc.bn, (cudaStream_t)stream);
}

// General form of the three entry points above, plus a LayerNorm folded in on the input side and
// per-row statistics on the output side.
extern "C" int bxl_gemm_fused_f16(const bxl_gemm_fused_args* a, int* row_stats_parts, void* stream) {
  if (!a) return fail(kErrInvalidArg, "bxl_gemm_fused_f16: null argument block");
  const int M = a->M, N = a->N, K = a->K;
  if (!a->A || !a->B || !a->C) return fail(kErrInvalidArg, "bxl_gemm_fused_f16: null operand");
  if (M <= 0 || N <= 0 || K <= 0) return fail(kErrInvalidArg, "bxl_gemm_fused_f16: non-positive extent M=%d N=%d K=%d", M, N, K);
  if (a->lda % 8 || a->ldb % 8 || a->lda < K || a->ldb < K) return fail(kErrInvalidArg, "bxl_gemm_fused_f16: bad lda/ldb");
  if (!aligned16(a->A) || !aligned16(a->B) || !aligned16(a->C) || (a->residual && !aligned16(a->residual)) || (a->C2 && !aligned16(a->C2)))
    return fail(kErrInvalidArg, "bxl_gemm_fused_f16: operands must be 16-byte aligned");
  if (a->geglu && (N % 32 || a->n_split || a->residual || a->row_stats))
    return fail(kErrInvalidArg, "bxl_gemm_fused_f16: the GEGLU epilogue needs N %% 32 == 0 and excludes a second destination, a residual and row statistics");
  const int n_out = a->geglu ? N / 2 : N;
  if (a->n_split) {
    if (!a->C2 || a->n_split <= 0 || a->n_split >= N || a->n_split % 32 || N % 8 || a->residual || a->row_stats)
      return fail(kErrInvalidArg, "bxl_gemm_fused_f16: second destination needs 0 < n_split < N, n_split %% 32 == 0, no residual, no row statistics");
    if (a->ldc % 8 || a->ldc2 % 8 || a->ldc < a->n_split || a->ldc2 < N - a->n_split) return fail(kErrInvalidArg, "bxl_gemm_fused_f16: bad ldc/ldc2");
  } else if (a->ldc % 8 || a->ldc < n_out) {
    return fail(kErrInvalidArg, "bxl_gemm_fused_f16: bad ldc");
  }
  if (a->residual && (a->ldr % 8 || a->ldr < N)) return fail(kErrInvalidArg, "bxl_gemm_fused_f16: bad ldr");
  const bool ln = a->ln_partials != nullptr;
  if (ln && (a->ln_parts <= 0 || !a->ln_colsum || !(a->ln_eps > 0.f) || (reinterpret_cast<uintptr_t>(a->ln_partials) & 7u)))
    return fail(kErrInvalidArg, "bxl_gemm_fused_f16: folded LayerNorm needs ln_parts > 0, column sums and a positive epsilon");
  if (a->row_stats && (N % 32 || !row_stats_parts || (reinterpret_cast<uintptr_t>(a->row_stats) & 7u)))
    return fail(kErrInvalidArg, "bxl_gemm_fused_f16: row statistics need N %% 32 == 0 and a place for the partial count");
  int* st = device_status_ptr();
  if (!st) return fail(kErrCuda, "bxl_gemm_fused_f16: no device status word");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const int tiles_m = (M + kBM - 1) / kBM;
  const TileConfig tc = choose_tiles(tiles_m, N, (K + kBK - 1) / kBK, false, g_force_bn, g_force_split,
                                     g_force_pair < 0 ? kDefaultPair : g_force_pair, 0.0, ln ? kSmemLnExtra : 0);
  const int tiles_n = (N + tc.bn - 1) / tc.bn;
  if (a->row_stats) {
    const long long parts = (long long)kEpiSub * tiles_n * (tc.pair ? 1 : tc.split);  // one per epilogue warp of a row and column slice
    if (a->row_stats_capacity < 2ll * M * parts)
      return fail(kErrTooLarge, "bxl_gemm_fused_f16: row statistics need %lld floats, %lld given", 2ll * M * parts, a->row_stats_capacity);
    *row_stats_parts = (int)parts;
    p.stat_out = reinterpret_cast<float2*>(a->row_stats);
    p.stat_parts = (int)parts;
  }
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t str[1] = {(uint64_t)a->lda * 2};
    uint32_t box[2] = {kBK, kBM};
    if (int rc = encode_tmap_f16(&p.a_map[0], a->A, 2, dims, str, box)) return rc;
  }
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)N};
    uint64_t str[1] = {(uint64_t)a->ldb * 2};
    uint32_t box[2] = {kBK, (uint32_t)(tc.pair ? tc.bn / 2 : tc.bn)};
    if (int rc = encode_tmap_f16(&p.b_map[0], a->B, 2, dims, str, box)) return rc;
  }
  for (int s = 1; s < kMaxSeg; ++s) {
    p.a_map[s] = p.a_map[0];
    p.b_map[s] = p.b_map[0];
  }
  p.M = M, p.N = N, p.K = K, p.nseg = 1, p.b_kn = 0;
  p.bn = tc.bn, p.split = tc.split, p.stages = tc.stages, p.pair = tc.pair, p.b_static = static_weights() ? 1 : 0;
  p.n_fastest = linear_tile_order(M, N, K, tc.bn);
  p.bias = static_cast<const __half*>(a->bias);
  p.bias_f32 = a->bias_f32;
  p.residual = static_cast<const __half*>(a->residual);
  p.ldr = a->ldr, p.C = a->C, p.ldc = a->ldc, p.C2 = a->C2, p.ldc2 = a->ldc2, p.n_split = a->n_split, p.geglu = a->geglu ? 1 : 0;
  if (ln) {
    p.ln_part = reinterpret_cast<const float2*>(a->ln_partials);
    p.ln_parts = a->ln_parts;
    p.ln_inv_k = 1.f / (float)K;
    p.ln_eps = a->ln_eps;
    p.ln_colsum = a->ln_colsum;
  }
  p.dev_status = st;
  return launch<false>(p, tiles_m, tiles_n, (cudaStream_t)stream);
}

extern "C" int bxl_debug_force_tiles(int bn, int split, int pair) {
  if (bn < 0 || bn > 256 || bn % 32 || (split != 0 && split != 1 && split != 2 && split != 4) || pair < -1 || pair > 1)
    return fail(kErrInvalidArg, "bxl_debug_force_tiles: bn must be 0 or a multiple of 32 up to 256, split 0, 1, 2 or 4, pair -1, 0 or 1");
  g_force_bn = bn, g_force_split = split, g_force_pair = pair;
  return kOk;
}

extern "C" int bxl_debug_force_tile_order(int order) {
  if (order < -1 || order > 1) return fail(kErrInvalidArg, "bxl_debug_force_tile_order: -1 (choose), 0 (walk M first) or 1 (walk N first)");
  g_force_order = order;
  return kOk;
}

// ---- split-operand product of fp32 matrices ---------------------------------------
namespace bxl {
// x = hi + lo with hi = fp16(x), lo = fp16(x - hi): 22 significant bits kept.
__global__ void split_f32_kernel(const float* __restrict__ x, __half* __restrict__ hi, __half* __restrict__ lo, long long n4) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n4; i += (long long)gridDim.x * blockDim.x) {
    const float4 v = reinterpret_cast<const float4*>(x)[i];
    const __half h0 = __float2half_rn(v.x), h1 = __float2half_rn(v.y), h2 = __float2half_rn(v.z), h3 = __float2half_rn(v.w);
    __half2 hh[2] = {__halves2half2(h0, h1), __halves2half2(h2, h3)};
    __half2 ll[2] = {__floats2half2_rn(v.x - __half2float(h0), v.y - __half2float(h1)),
                     __floats2half2_rn(v.z - __half2float(h2), v.w - __half2float(h3))};
    reinterpret_cast<uint2*>(hi)[i] = *reinterpret_cast<uint2*>(hh);
    reinterpret_cast<uint2*>(lo)[i] = *reinterpret_cast<uint2*>(ll);
  }
}
}  // namespace bxl

extern "C" long long bxl_gemm_split_workspace_bytes(int M, int N, int K) {
  if (M <= 0 || N <= 0 || K <= 0) return 0;
  return 2ll * 2 * ((long long)M * K + (long long)K * N) + 1024;
}

extern "C" int bxl_gemm_split_f32(const float* A, const float* B, float* C, int M, int N, int K, void* workspace,
                                  long long workspace_bytes, void* stream) {
  if (!A || !B || !C || !workspace) return fail(kErrInvalidArg, "bxl_gemm_split_f32: null pointer");
  if (M <= 0 || N <= 0 || K <= 0) return fail(kErrInvalidArg, "bxl_gemm_split_f32: non-positive extent");
  if (K % 8 || N % 8) return fail(kErrInvalidArg, "bxl_gemm_split_f32: K and N must be multiples of 8");
  if (!aligned16(A) || !aligned16(B) || !aligned16(C) || !aligned16(workspace))
    return fail(kErrInvalidArg, "bxl_gemm_split_f32: pointers must be 16-byte aligned");
  if (workspace_bytes < bxl_gemm_split_workspace_bytes(M, N, K)) return fail(kErrTooLarge, "bxl_gemm_split_f32: workspace too small");
  int* st = device_status_ptr();
  if (!st) return fail(kErrCuda, "bxl_gemm_split_f32: no device status word");
  cudaStream_t s = (cudaStream_t)stream;
  const long long na = (long long)M * K, nb = (long long)K * N;
  __half* a_hi = static_cast<__half*>(workspace);
  __half* a_lo = a_hi + na;
  __half* b_hi = a_lo + na;
  __half* b_lo = b_hi + nb;
  const int blocks = sm_count() * 8;
  split_f32_kernel<<<blocks, 256, 0, s>>>(A, a_hi, a_lo, na / 4);
  split_f32_kernel<<<blocks, 256, 0, s>>>(B, b_hi, b_lo, nb / 4);
  if (int rc = check_cuda(cudaGetLastError(), "split_f32_kernel launch")) return rc;
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const int tiles_m = (M + kBM - 1) / kBM;
  const TileConfig tc = choose_tiles(tiles_m, N, 3 * ((K + kBK - 1) / kBK), true, g_force_bn, g_force_split, g_force_pair < 0 ? kDefaultPair : g_force_pair);
  const int BN = tc.bn;
  // C = A_hi*B_hi + A_hi*B_lo + A_lo*B_hi, one fp32 accumulator
  const __half* as[3] = {a_hi, a_hi, a_lo};
  const __half* bs[3] = {b_hi, b_lo, b_hi};
  for (int i = 0; i < 3; ++i) {
    uint64_t ad[2] = {(uint64_t)K, (uint64_t)M};
    uint64_t astr[1] = {(uint64_t)K * 2};
    uint32_t abox[2] = {kBK, kBM};
    if (int rc = encode_tmap_f16(&p.a_map[i], as[i], 2, ad, astr, abox)) return rc;
    uint64_t bd[2] = {(uint64_t)N, (uint64_t)K};
    uint64_t bstr[1] = {(uint64_t)N * 2};
    uint32_t bbox[2] = {64, kBK};
    if (int rc = encode_tmap_f16(&p.b_map[i], bs[i], 2, bd, bstr, bbox)) return rc;
  }
  p.M = M, p.N = N, p.K = K, p.nseg = 3, p.b_kn = 1;
  // b_static stays 0: the fp16 parts of B were written by the kernel launched just above
  p.bn = tc.bn, p.split = tc.split, p.stages = tc.stages, p.pair = tc.pair;
  p.C = C, p.ldc = N, p.out_f32 = 1;
  p.dev_status = st;
  return launch<false>(p, tiles_m, (N + BN - 1) / BN, s);
}

// ---- convolution --------------------------------------------------------------------
namespace bxl {
// [C_out][C_in][3][3] -> [C_out][ky][kx][C_in]  (K index = tap*C_in + c)
__global__ void conv_weight_pack_kernel(const __half* __restrict__ w, __half* __restrict__ out, int cout, int cin) {
  // No early release of the successor: a convolution launched right after this kernel may fetch
  // the packed weights before its own grid-dependency wait (static-weights mode), so it must not
  // start before every store below has completed.
  pdl_wait();
  const long long total = (long long)cout * cin * 9;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int c = i % cin;
    const int tap = (i / cin) % 9;
    const int o = i / (9ll * cin);
    out[i] = w[((long long)o * cin + c) * 9 + tap];
  }
}
}  // namespace bxl

extern "C" int bxl_conv_weight_pack_f16(const void* w_oihw, void* w_packed, int c_out, int c_in, void* stream) {
  if (!w_oihw || !w_packed || c_out <= 0 || c_in <= 0) return fail(kErrInvalidArg, "bxl_conv_weight_pack_f16: bad argument");
  conv_weight_pack_kernel<<<sm_count() * 4, 256, 0, (cudaStream_t)stream>>>(static_cast<const __half*>(w_oihw),
                                                                             static_cast<__half*>(w_packed), c_out, c_in);
  return check_cuda(cudaGetLastError(), "conv_weight_pack_kernel launch");
}

extern "C" int bxl_conv3x3_halo_f16(const void* x, long long x_img_stride, const void* top, const void* bot,
                                    long long halo_img_stride, const void* w_packed, const void* bias, const void* bias_rows,
                                    long long bias_rows_stride, const void* residual, void* y, int B, int C_in, int C_out,
                                    int H_in, int W, int stride, void* stream) {
  if (!x || !w_packed || !y) return fail(kErrInvalidArg, "bxl_conv3x3_halo_f16: null operand");
  if (B <= 0 || H_in <= 0 || W <= 0) return fail(kErrInvalidArg, "bxl_conv3x3_halo_f16: non-positive extent");
  if (stride != 1 && stride != 2) return fail(kErrUnsupported, "bxl_conv3x3_halo_f16: stride %d (1 or 2 supported)", stride);
  if (C_in % 64) return fail(kErrUnsupported, "bxl_conv3x3_halo_f16: C_in=%d must be a multiple of 64 (use the direct kernel)", C_in);
  if (C_out % 4) return fail(kErrUnsupported, "bxl_conv3x3_halo_f16: C_out=%d must be a multiple of 4", C_out);
  if (W % stride || H_in % stride) return fail(kErrInvalidArg, "bxl_conv3x3_halo_f16: H and W must be multiples of the stride");
  if (!aligned16(x) || !aligned16(w_packed) || !aligned16(y) || (top && !aligned16(top)) || (bot && !aligned16(bot)) ||
      (residual && !aligned16(residual)))
    return fail(kErrInvalidArg, "bxl_conv3x3_halo_f16: pointers must be 16-byte aligned");
  if (x_img_stride % 8 || halo_img_stride % 8) return fail(kErrInvalidArg, "bxl_conv3x3_halo_f16: image strides must be multiples of 8");
  if (bias_rows && bias_rows_stride != 0 && bias_rows_stride < C_out)
    return fail(kErrInvalidArg, "bxl_conv3x3_halo_f16: bias_rows_stride=%lld is smaller than C_out=%d", bias_rows_stride, C_out);
  int* st = device_status_ptr();
  if (!st) return fail(kErrCuda, "bxl_conv3x3_halo_f16: no device status word");
  GemmParams p;
  memset(&p, 0, sizeof(p));
  const int Wh = W / stride;  // half-columns (== output width)
  const int H_out = H_in / stride, W_out = W / stride;
  int tw = 128;
  while (tw > W_out && tw > 8) tw >>= 1;  // tile width: power of two <= W_out, >= 8
  const int th = 128 / tw;
  // 5-D view [C, stride, W/stride, H, B] of an NHWC strip
  auto enc = [&](CUtensorMap* m, const void* base, int rows, long long img_stride) {
    uint64_t dims[5] = {(uint64_t)C_in, (uint64_t)stride, (uint64_t)Wh, (uint64_t)rows, (uint64_t)B};
    uint64_t str[4] = {(uint64_t)C_in * 2, (uint64_t)stride * C_in * 2, (uint64_t)W * C_in * 2, (uint64_t)img_stride * 2};
    uint32_t box[5] = {kBK, 1, (uint32_t)tw, 1, 1};
    return encode_tmap_f16(m, base, 5, dims, str, box);
  };
  if (int rc = enc(&p.a_map[0], x, H_in, x_img_stride)) return rc;
  {
    uint64_t dims[5] = {(uint64_t)C_in, (uint64_t)stride, (uint64_t)Wh, (uint64_t)H_in, (uint64_t)B};
    uint64_t str[4] = {(uint64_t)C_in * 2, (uint64_t)stride * C_in * 2, (uint64_t)W * C_in * 2, (uint64_t)x_img_stride * 2};
    uint32_t box[5] = {kBK, 1, (uint32_t)tw, (uint32_t)th, 1};
    if (int rc = encode_tmap_f16(&p.a_rows_map, x, 5, dims, str, box)) return rc;
  }
  if (int rc = enc(&p.a_map[1], top ? top : x, 1, top ? halo_img_stride : x_img_stride)) return rc;
  if (int rc = enc(&p.a_map[2], bot ? bot : x, 1, bot ? halo_img_stride : x_img_stride)) return rc;
  const int K = 9 * C_in;
  const int tiles_x = (W_out + tw - 1) / tw, tiles_y = (H_out + th - 1) / th;
  const TileConfig tc = choose_tiles(B * tiles_x * tiles_y, C_out, K / kBK, false, g_force_bn, g_force_split,
                                     g_force_pair < 0 ? kDefaultPair : g_force_pair, kConvAMinUs);
  const int BN = tc.bn;
  {
    uint64_t dims[2] = {(uint64_t)K, (uint64_t)C_out};
    uint64_t str[1] = {(uint64_t)K * 2};
    uint32_t box[2] = {kBK, (uint32_t)(tc.pair ? BN / 2 : BN)};
    if (int rc = encode_tmap_f16(&p.b_map[0], w_packed, 2, dims, str, box)) return rc;
  }
  p.b_map[1] = p.b_map[0];
  p.b_map[2] = p.b_map[0];
  p.M = B * H_out * W_out, p.N = C_out, p.K = K, p.nseg = 1, p.b_kn = 0;
  p.bn = tc.bn, p.split = tc.split, p.stages = tc.stages, p.pair = tc.pair, p.b_static = static_weights() ? 1 : 0;
  p.bias = static_cast<const __half*>(bias);
  p.bias_rows = static_cast<const __half*>(bias_rows);
  p.ld_bias_rows = bias_rows_stride > 0 ? bias_rows_stride : C_out;
  p.residual = static_cast<const __half*>(residual);
  p.ldr = C_out, p.C = y, p.ldc = C_out, p.out_f32 = 0;
  p.cB = B, p.cHin = H_in, p.cW = W, p.cCin = C_in, p.cStride = stride, p.cHout = H_out, p.cWout = W_out;
  p.tw = tw, p.th = th;
  p.tiles_x = tiles_x, p.tiles_y = tiles_y;
  p.has_top = top ? 1 : 0, p.has_bot = bot ? 1 : 0;
  // An input that does not stay in L2 while the output streams through it is walked once: the CTAs
  // running at the same time then take the column tiles of the same pixels (the packed weights,
  // a few MB, stay resident instead).
  p.n_fastest = (C_out > BN && 2ll * B * H_in * W * C_in > (48ll << 20)) ? 1 : 0;
  if (g_force_order >= 0) p.n_fastest = g_force_order;
  p.dev_status = st;
  return launch<true>(p, B * tiles_x * tiles_y, (C_out + BN - 1) / BN, (cudaStream_t)stream);
}

extern "C" int bxl_set_static_weights(int enabled) {
  set_static_weights(enabled != 0);
  return kOk;
}
