// Flash-style attention for sm_100a on tcgen05 / TMEM: the local queries of one
// strip against the full key/value sequence, which lives as up to 8 per-peer
// slots [B, L_slot, 2C] (K in columns [0,C), V in [C,2C), head h at columns
// h*64..h*64+63).  The slots are read IN PLACE through one TMA descriptor per
// slot: the own strip's fresh K/V and the peers' stale K/V are never
// concatenated.  The same kernel serves cross-attention (one slot, 77 tokens).
//
// Work unit = 256 queries (two tiles of 128) of one (image, head).  A CTA walks several units
// (or, with a K/V split, a cluster of 2 or 4 CTAs shares one unit).  384 threads:
//   warps 0..3  softmax group 0, warps 4..7 softmax group 1: thread r owns query row r of its
//               tile (= TMEM lane r).  Per K/V tile it reads its row of S once (128 registers),
//               releases S at once so the next Q K^T can start, takes the row maximum, forms
//               P = exp2(S*scale - m) in fp32 (MUFU), sums the row in fp32 registers, packs P to
//               fp16 and stores it to TENSOR MEMORY (tcgen05.st), from where the P V product
//               reads it as its A operand: P never touches shared memory.  The running maximum
//               m is only raised when the tile maximum exceeds it by more than 8 (a factor of
//               256, harmless in fp16/fp32); only then O is rescaled in tensor memory
//               (tcgen05.ld / multiply / tcgen05.st) and the row sum in its register.  The
//               result is exact: O and the row sum always refer to the same m.
//               These two warpgroups raise their register budget (setmaxnreg) at the expense
//               of the third one.
//   warp 8      TMA producer: the two Q tiles of a unit (double buffered across units), then a
//               ring of {K tile, V tile} (128 tokens x 64) shared by the two query tiles
//   warp 9      tensor memory owner and tcgen05.mma issuer (all 32 lanes run the loop, an
//               elected lane issues), for the two query tiles g = 0, 1:
//                 S_g  = Q_g K_j^T      (128x128, both operands K-major in shared memory)
//                 O_g += P_g V_j        (128x64, P from tensor memory, V MN-major as stored)
//               issued in the order in which their conditions come true.
//   warps 10,11 idle (they complete the third warpgroup).
// While one group runs its softmax the tensor core works for the other one; the K/V tiles of
// all units of a CTA form one stream, so the first Q K^T of the next unit and the read-out of
// the finished unit's output overlap the unit boundary.
//
// Roofline: tensor cores; algorithmic FLOPs = 4 * L_q * L_kv * 64 per (image, head).
// With head dimension 64 the softmax side (one MUFU exponential plus ~3 more instructions per
// score, two warps per scheduler) needs more cycles per tile than the two matrix products;
// measured, the kernel is bound by that instruction stream (evaluating part of the
// exponentials with a polynomial on the FMA pipe made it slower).
#include <stdlib.h>

#include "bxl_common.cuh"
#include "bxl_host.h"
#include "../../include/basedxl_b200.h"

namespace bxl {

constexpr int kAttnThreads = 384;   // warps 0..7 softmax, 8 producer, 9 MMA issuer, 10..11 idle
constexpr int kSoftmaxRegs = 208;   // registers per thread after the split: 8 x 32 x 208 + 4 x 32 x 88 = 64512
constexpr int kOtherRegs = 88;
constexpr int kHeadDim = 64;
constexpr int kTileQ = 128;
constexpr int kTileKV = 128;
constexpr int kKvStages = 4;
constexpr int kMaxSlots = 8;

struct alignas(64) AttnParams {
  CUtensorMap q_map;               // [C_q cols, L_q, B]
  CUtensorMap kv_map[kMaxSlots];   // [2C cols, L_slot, B] per slot
  int n_slots;
  int L_q, L_slot;
  int heads, B;
  int v_col0;                      // column of V for head 0 (= C)
  __half* out;                     // [B, L_q, ld_out]
  long long out_img_stride, ld_out;
  float scale_log2e;               // softmax scale * log2(e)
  int kv_split;                    // K/V range split over a cluster of 1, 2 or 4 CTAs
  int n_full;                      // units [0, n_full) are whole (256 queries); each later unit is served as two halves of 128
  int* dev_status;
};

struct AttnSmem {
  static constexpr int kQ = 0;                               // 2 buffers x 2 tiles x 16 KB
  static constexpr int kK = 65536;                           // kKvStages x 16 KB
  static constexpr int kV = kK + kKvStages * 16384;          // kKvStages x 16 KB
  static constexpr int kBar = kV + kKvStages * 16384;
  static constexpr int kTotal = kBar + 1024 + 1024;
};

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}
__device__ __forceinline__ uint32_t pack_f16x2(float a, float b) {
  uint32_t packed;
  asm("cvt.rn.f16x2.f32 %0, %1, %2;" : "=r"(packed) : "f"(b), "f"(a));
  return packed;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ void tmem_st_32x32(uint32_t taddr, const uint32_t (&r)[32]) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16, "
      "%17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31, %32};" ::"r"(taddr),
      "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]), "r"(r[10]),
      "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15]), "r"(r[16]), "r"(r[17]), "r"(r[18]), "r"(r[19]), "r"(r[20]),
      "r"(r[21]), "r"(r[22]), "r"(r[23]), "r"(r[24]), "r"(r[25]), "r"(r[26]), "r"(r[27]), "r"(r[28]), "r"(r[29]), "r"(r[30]),
      "r"(r[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
// Ragged last tile of a slot, one 32-column chunk with nv valid columns (warp-uniform): row
// maximum, and P = exp2(s*sc - m) packed into pk[kOff .. kOff+15] with its sum.  Chunks without
// a valid column cost nothing.
__device__ __forceinline__ float ragged_chunk_max(const uint32_t (&v)[32], int nv) {
  float m = -INFINITY;
  if (nv >= 32) {
    float m2 = -INFINITY;
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      m = max3(m, __uint_as_float(v[i]), __uint_as_float(v[i + 1]));
      m2 = max3(m2, __uint_as_float(v[i + 2]), __uint_as_float(v[i + 3]));
    }
    m = fmaxf(m, m2);
  } else if (nv > 0) {
#pragma unroll
    for (int i = 0; i < 32; ++i)
      if (i < nv) m = fmaxf(m, __uint_as_float(v[i]));
  }
  return m;
}
template <int kOff>
__device__ __forceinline__ float ragged_chunk_p(const uint32_t (&v)[32], uint32_t (&pk)[32], int nv, float sc, float m) {
  float s0 = 0.f, s1 = 0.f;
  if (nv >= 32) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float a = fast_exp2(fmaf(__uint_as_float(v[2 * i]), sc, -m)), b = fast_exp2(fmaf(__uint_as_float(v[2 * i + 1]), sc, -m));
      s0 += a, s1 += b;
      pk[kOff + i] = pack_f16x2(a, b);
    }
  } else if (nv > 0) {
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const float a = (2 * i < nv) ? fast_exp2(fmaf(__uint_as_float(v[2 * i]), sc, -m)) : 0.f;
      const float b = (2 * i + 1 < nv) ? fast_exp2(fmaf(__uint_as_float(v[2 * i + 1]), sc, -m)) : 0.f;
      s0 += a, s1 += b;
      pk[kOff + i] = pack_f16x2(a, b);
    }
  } else {
#pragma unroll
    for (int i = 0; i < 16; ++i) pk[kOff + i] = 0u;
  }
  return s0 + s1;
}

// One query row of a finished unit: read O (64 fp32 columns of this thread's TMEM lane),
// normalise by the row sum and store 64 halves.  Kept out of line: it is called from inside the
// K/V loop, where the registers are needed for the row of S.
__device__ __noinline__ void attn_store_row(uint32_t o_addr, __half* dst, float inv_l) {
  uint32_t o0[32], o1[32];
  tmem_ld_32x32(o_addr, o0);
  tmem_ld_32x32(o_addr + 32, o1);
  tmem_ld_wait();
  if (dst == nullptr) return;
  // 128 bytes of this thread's output row: four whole 32-byte sectors when the row is aligned
  uint32_t w[32];
#pragma unroll
  for (int j = 0; j < 16; ++j) {
    w[j] = pack_f16x2(__uint_as_float(o0[2 * j]) * inv_l, __uint_as_float(o0[2 * j + 1]) * inv_l);
    w[16 + j] = pack_f16x2(__uint_as_float(o1[2 * j]) * inv_l, __uint_as_float(o1[2 * j + 1]) * inv_l);
  }
  if ((reinterpret_cast<uintptr_t>(dst) & 31u) == 0) {
#pragma unroll
    for (int q = 0; q < 4; ++q)
      st_global_v8(dst + q * 16, w[8 * q], w[8 * q + 1], w[8 * q + 2], w[8 * q + 3], w[8 * q + 4], w[8 * q + 5], w[8 * q + 6],
                   w[8 * q + 7]);
  } else {
#pragma unroll
    for (int q = 0; q < 8; ++q) *reinterpret_cast<uint4*>(dst + q * 8) = make_uint4(w[4 * q], w[4 * q + 1], w[4 * q + 2], w[4 * q + 3]);
  }
}

__global__ void __launch_bounds__(kAttnThreads, 1) attention_kernel(const __grid_constant__ AttnParams p) {
  extern __shared__ uint8_t smem_raw[];
  const uint32_t smem_base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* smem_gen = smem_raw + (smem_base - smem_u32(smem_raw));
  const uint32_t bar_base = smem_base + AttnSmem::kBar;
  // barriers: q_full[2], q_empty[2], kv_full[stages], kv_empty[stages], s_full[2], o_full[2], p_full[2], s_free[2]
  auto q_full = [&](int b) { return bar_base + 8u * b; };
  auto q_empty = [&](int b) { return bar_base + 8u * (2 + b); };
  auto kv_full = [&](int s) { return bar_base + 8u * (4 + s); };
  auto kv_empty = [&](int s) { return bar_base + 8u * (4 + kKvStages + s); };
  auto s_full = [&](int g) { return bar_base + 8u * (4 + 2 * kKvStages + g); };
  auto o_full = [&](int g) { return bar_base + 8u * (6 + 2 * kKvStages + g); };
  auto p_full = [&](int g) { return bar_base + 8u * (8 + 2 * kKvStages + g); };
  auto s_free = [&](int g) { return bar_base + 8u * (10 + 2 * kKvStages + g); };
  volatile uint32_t* tmem_slot = reinterpret_cast<volatile uint32_t*>(smem_gen + AttnSmem::kBar + 512);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(smem_gen + AttnSmem::kBar + 520);

  pdl_launch_dependents();
  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  // S_0 [0,128) S_1 [128,256) O_0 [256,320) O_1 [320,384) P_0 [384,448) P_1 [448,512)
  // (P: 128 fp16 per row packed two per 32-bit column, the A operand of the P V product)
  constexpr uint32_t kTmemCols = 512;

  // Work units: 256 queries (two tiles) of one (image, head).
  //   kv_split == 1: the CTA walks units blockIdx.x, blockIdx.x + gridDim.x, ...; barriers, the
  //     K/V ring and tensor memory live across units, Q is double buffered, so the loads and the
  //     first Q K^T of the next unit overlap the tail of the current one.
  //   kv_split == S > 1: the S CTAs of a cluster serve ONE unit, each over 1/S of the K/V tiles;
  //     their partial (max, sum, output) triples are merged through distributed shared memory at
  //     the end (every CTA merges 256/S of the rows).
  const int S = p.kv_split;
  const uint32_t crank = (S > 1) ? cluster_ctarank() : 0u;
  const int q_pairs = (p.L_q + 2 * kTileQ - 1) / (2 * kTileQ);
  // Units past n_full are the last, under-filled round of a persistent grid: each is served as two
  // half units (one query tile) so that twice as many CTAs share that round.
  const int n_full = p.n_full;
  const int units_total = n_full + 2 * (q_pairs * p.heads * p.B - n_full);
  const int first_unit = (S > 1) ? static_cast<int>(blockIdx.x) / S : static_cast<int>(blockIdx.x);
  const int unit_step = (S > 1) ? units_total : static_cast<int>(gridDim.x);
  auto unit_pair = [&](int w) { return w < n_full ? w : n_full + ((w - n_full) >> 1); };      // index of the 256-query block
  auto unit_q_row0 = [&](int w) { return (unit_pair(w) % q_pairs) * 2 * kTileQ + ((w >= n_full && ((w - n_full) & 1)) ? kTileQ : 0); };
  auto unit_head = [&](int w) { return (unit_pair(w) / q_pairs) % p.heads; };
  auto unit_img = [&](int w) { return unit_pair(w) / (q_pairs * p.heads); };
  // the second tile may lie wholly past L_q; a half unit has one tile
  auto unit_groups = [&](int w) { return (w < n_full && unit_q_row0(w) + kTileQ < p.L_q) ? 2 : 1; };
  const int tiles_per_slot = (p.L_slot + kTileKV - 1) / kTileKV;
  const int total_tiles = p.n_slots * tiles_per_slot;
  const int tile0 = static_cast<int>((static_cast<long long>(crank) * total_tiles) / S);   // first K/V tile of this CTA
  const int n_tiles = static_cast<int>((static_cast<long long>(crank + 1) * total_tiles) / S) - tile0;
  // kv_split > 1 only: per-thread result of the K/V loop (softmax threads), kept for the merge
  uint32_t fin_o[kHeadDim];
  float fin_l = 0.f, fin_m = -INFINITY;
  bool fin_valid = false;

  if (threadIdx.x == 0) {
    for (int b = 0; b < 2; ++b) {
      mbar_init(q_full(b), 1);
      mbar_init(q_empty(b), 1);
    }
    for (int s = 0; s < kKvStages; ++s) {
      mbar_init(kv_full(s), 1);
      mbar_init(kv_empty(s), 1);
    }
    for (int g = 0; g < 2; ++g) {
      mbar_init(s_full(g), 1);
      mbar_init(o_full(g), 1);
      mbar_init(p_full(g), 128);
      mbar_init(s_free(g), 128);
    }
    *abort_flag = 0;
    mbar_fence_init();
  }
  if (warp == 9) {
    tmem_alloc(smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
    tmem_relinquish();
  }
  tc_fence_before_sync();
  __syncthreads();
  tc_fence_after_sync();
  const uint32_t tmem_base = *tmem_slot;
  // the softmax warps hold a whole row of S (128 values) and of P: give them the registers the
  // producer / MMA warpgroup does not need
  pdl_wait();  // the set-up above overlaps the previous kernel's tail; global data from here on

  if (warp >= 8) {
  asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(kOtherRegs));
  if (warp == 8) {
    // ======================= TMA producer =======================
    // all 32 lanes run the loop (addresses stay warp-uniform); the elected lane issues
    const bool leader = elect_one();
    if (leader) tma_prefetch_desc(&p.q_map);
    __syncwarp();
    int stage = 0;
    uint32_t phase = 0;
    bool ok = true;
    int ul = 0;  // units started by this CTA
    for (int w = first_unit; w < units_total && ok; w += unit_step, ++ul) {
      const int qb = ul & 1;
      const int ng = unit_groups(w);
      const int head = unit_head(w), img = unit_img(w), q_row0 = unit_q_row0(w);
      // the Q buffer was last used by unit ul - 2: all its Q K^T products must have completed
      if (ul >= 2 && !mbar_wait_warp(q_empty(qb), ((ul >> 1) - 1) & 1u, abort_flag, p.dev_status, 401)) break;
      if (leader) {
        mbar_arrive_expect_tx(q_full(qb), 16384u * ng);
        for (int g = 0; g < ng; ++g)
          tma_load_3d(smem_base + AttnSmem::kQ + qb * 32768 + g * 16384, &p.q_map, q_full(qb), head * kHeadDim,
                      q_row0 + g * kTileQ, img);
      }
      __syncwarp();
      for (int j = 0; j < n_tiles; ++j) {
        const int slot = (tile0 + j) / tiles_per_slot;
        const int t0 = ((tile0 + j) % tiles_per_slot) * kTileKV;
        if (!mbar_wait_warp(kv_empty(stage), phase ^ 1u, abort_flag, p.dev_status, 400)) {
          ok = false;
          break;
        }
        if (leader) {
          mbar_arrive_expect_tx(kv_full(stage), 32768);
          tma_load_3d(smem_base + AttnSmem::kK + stage * 16384, &p.kv_map[slot], kv_full(stage), head * kHeadDim, t0, img);
          tma_load_3d(smem_base + AttnSmem::kV + stage * 16384, &p.kv_map[slot], kv_full(stage),
                      p.v_col0 + head * kHeadDim, t0, img);
        }
        __syncwarp();
        if (++stage == kKvStages) {
          stage = 0;
          phase ^= 1u;
        }
      }
    }
  } else if (warp == 9) {
    // ======================= MMA issuer =======================
    // all 32 lanes run the loop and the waits; the elected lane issues every tcgen05.mma and
    // tcgen05.commit, so descriptors are formed from warp-uniform values.  The K/V tiles of all
    // units of this CTA form one stream: while the softmax of tile t runs, Q K^T of tile t+1 is
    // issued, also across a unit boundary.
    const bool leader = elect_one();
    const uint32_t idesc_s = make_idesc_f16(128, 128, 0, 0);  // S = Q K^T, both K-major
    const uint32_t idesc_o = make_idesc_f16(128, 64, 0, 1);   // O = P V, V MN-major
    int n_s[2] = {0, 0};   // Q K^T products issued per group (= phases of s_full started)
    int n_pv[2] = {0, 0};  // P V products issued per group
    int kv_t = 0;          // K/V tiles of the stream consumed so far
    bool ok = true;
    auto wait_kv = [&](int t) -> bool {
      if (!mbar_wait_warp(kv_full(t % kKvStages), (t / kKvStages) & 1u, abort_flag, p.dev_status, 501)) return false;
      tc_fence_after_sync();
      return true;
    };
    // S_g = Q_g K^T for stream tile t of the unit in Q buffer qb; S_g must have been read by the
    // softmax group (s_free) if it was ever written
    auto issue_s = [&](int qb, int g, int t) -> bool {
      if (n_s[g] > 0) {
        if (!mbar_wait_warp(s_free(g), (n_s[g] - 1) & 1u, abort_flag, p.dev_status, 503)) return false;
        tc_fence_after_sync();
      }
      const int st = t % kKvStages;
      const uint64_t qdesc = make_smem_desc_sw128(smem_base + AttnSmem::kQ + qb * 32768 + g * 16384, 16, 1024);
      const uint64_t kdesc = make_smem_desc_sw128(smem_base + AttnSmem::kK + st * 16384, 16, 1024);
      const uint32_t d = tmem_base + g * 128;
      if (leader) {
#pragma unroll
        for (int k = 0; k < kHeadDim / 16; ++k) umma_f16(d, qdesc + 2u * k, kdesc + 2u * k, idesc_s, k != 0);
        umma_commit(s_full(g));
      }
      __syncwarp();
      ++n_s[g];
      return true;
    };
    int ul = 0;
    if (first_unit < units_total) {
      // first tile of the first unit
      ok = mbar_wait_warp(q_full(0), 0, abort_flag, p.dev_status, 500) && wait_kv(0);
      for (int g = 0; g < unit_groups(first_unit) && ok; ++g) ok = issue_s(0, g, 0);
    }
    for (int w = first_unit; w < units_total && ok; w += unit_step, ++ul) {
      const int qb = ul & 1;
      const int ng = unit_groups(w);
      const int w_next = w + unit_step;
      const bool has_next_unit = w_next < units_total;
      for (int j = 0; j < n_tiles && ok; ++j, ++kv_t) {
        const int st = kv_t % kKvStages;
        // tokens of this tile that exist (the last tile of a slot may be ragged): P is zero beyond
        // them, so their 16-token steps of the P V product are skipped
        const int k_steps = (min(kTileKV, p.L_slot - ((tile0 + j) % tiles_per_slot) * kTileKV) + 15) / 16;
        // V tile [128 tokens][64] as stored: MN-major B operand, 8-token groups 1 KB apart
        const uint64_t vdesc = make_smem_desc_sw128(smem_base + AttnSmem::kV + st * 16384, 16, 1024);
        // the tile after this one in the stream
        int nxt_ng = 0, nxt_qb = qb;
        if (j + 1 < n_tiles) {
          nxt_ng = ng;
        } else {
          // every Q K^T of this unit has been issued: its Q buffer is free once they complete
          if (leader) umma_commit(q_empty(qb));
          __syncwarp();
          if (has_next_unit) {
            nxt_ng = unit_groups(w_next), nxt_qb = qb ^ 1;
            if (!mbar_wait_warp(q_full(nxt_qb), ((ul + 1) >> 1) & 1u, abort_flag, p.dev_status, 500)) {
              ok = false;
              break;
            }
          }
        }
        if (nxt_ng > 0 && !wait_kv(kv_t + 1)) {
          ok = false;
          break;
        }
        // Four things are due for this tile: Q K^T of the next tile (per group, once the group
        // has copied its S) and P V of this tile (per group, once its P is published).  They are
        // issued in the order in which their conditions come true, so a late group never holds
        // up the other one.
        bool due_s[2] = {nxt_ng > 0, nxt_ng > 1};
        bool due_pv[2] = {ng > 0, ng > 1};
        const unsigned long long t_start = global_timer_ns();
        uint32_t spins = 0;
        while (due_s[0] || due_s[1] || due_pv[0] || due_pv[1]) {
          bool progress = false;
#pragma unroll
          for (int g = 0; g < 2; ++g) {
            if (due_s[g]) {
              const bool ready = (n_s[g] == 0) || __all_sync(0xffffffffu, mbar_try_wait(s_free(g), (n_s[g] - 1) & 1u));
              if (ready) {
                ok = issue_s(nxt_qb, g, kv_t + 1);  // its own wait on s_free returns at once
                due_s[g] = false, progress = true;
              }
            }
            if (due_pv[g] && __all_sync(0xffffffffu, mbar_try_wait(p_full(g), n_pv[g] & 1u))) {
              // P_g of this tile is in tensor memory; O_g carries the right scale
              tc_fence_after_sync();
              const uint32_t d = tmem_base + 256 + g * 64;
              const uint32_t pt = tmem_base + 384 + g * 64;
              const uint32_t acc = (j != 0);
              if (leader) {
#pragma unroll
                for (int k = 0; k < kTileKV / 16; ++k) {
                  // tokens 16k..16k+15: 8 packed columns of P, V rows advance by 16 x 128 B
                  if (k < k_steps) umma_f16_ts(d, pt + 8u * k, vdesc + 128u * k, idesc_o, acc | k);
                }
                umma_commit(o_full(g));
              }
              __syncwarp();
              ++n_pv[g];
              due_pv[g] = false, progress = true;
            }
          }
          if (!ok) break;
          if (!progress && (++spins & 63u) == 0u) {
            // bounded: give up after the common wait limit and report where
            bool give_up = (*abort_flag != 0);
            if (!give_up && global_timer_ns() - t_start > kWaitLimitNs) {
              give_up = true;
              *abort_flag = 1;
              if (atomicCAS(&p.dev_status[0], kDevOk, kDevWaitTimeout) == kDevOk) {
                p.dev_status[1] = 502;
                p.dev_status[2] = static_cast<int>(blockIdx.x);
              }
              __threadfence();
            }
            if (__any_sync(0xffffffffu, give_up)) {
              ok = false;
              break;
            }
          }
        }
        if (!ok) break;
        // K and V of this tile are no longer needed once everything issued so far has completed
        if (ok) {
          if (leader) umma_commit(kv_empty(st));
          __syncwarp();
        }
      }
    }
  }
    // producer / MMA warpgroup: the barriers of the hand-over, nothing to merge
    tc_fence_before_sync();
    __syncthreads();
    if (S > 1) {
      cluster_sync_all();
      cluster_sync_all();
    }
  } else {
    // ======================= softmax / output (warps 0..7) =======================
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(kSoftmaxRegs));
    const int g = warp >> 2;               // query tile served by this warp
    const int quarter = warp & 3;          // TMEM lane quarter this warp may access
    const int row = quarter * 32 + lane;   // query row inside the tile == TMEM lane
    const uint32_t t_lane = tmem_base + (static_cast<uint32_t>(quarter * 32) << 16);
    const uint32_t s_addr = t_lane + g * 128;
    const uint32_t o_addr = t_lane + 256 + g * 64;
    const uint32_t p_addr = t_lane + 384 + g * 64;
    const float sc = p.scale_log2e;
    constexpr float kRaise = 8.f;  // raise m only when the tile maximum exceeds it by 2^8
    int cnt = 0;                   // K/V tiles this group has processed (all units)
    bool ok = true;
    // The output of a finished unit stays in O_g while the first tile of the next unit is being
    // exponentiated; it is read out and stored just before that tile's P is published (the P V
    // product that would overwrite O_g is only issued after that).
    int pend_w = -1;             // unit whose output is still in tensor memory
    float pend_l = 1.f, pend_m = 0.f;
    // wait for the last P V product of the pending unit (tile cnt - 1), then store / keep its rows
    auto emit_pending = [&]() -> bool {
      if (!mbar_wait(o_full(g), (cnt - 1) & 1u, abort_flag, p.dev_status, 602)) return false;
      __syncwarp();
      tc_fence_after_sync();
      const int q_row = unit_q_row0(pend_w) + g * kTileQ + row;
      __half* dst = (q_row < p.L_q) ? p.out + (long long)unit_img(pend_w) * p.out_img_stride + (long long)q_row * p.ld_out +
                                          unit_head(pend_w) * kHeadDim
                                    : nullptr;
      attn_store_row(o_addr, dst, 1.f / pend_l);
      pend_w = -1;
      return true;
    };
    for (int w = first_unit; w < units_total && ok; w += unit_step) {
      if (g >= unit_groups(w)) continue;
      float m_run = -INFINITY;   // running row maximum in the exp2 domain (score * scale * log2 e)
      float l_run = 0.f;         // running row sum of P, same reference as O
      for (int j = 0; j < n_tiles && ok; ++j, ++cnt) {
        const int t0 = ((tile0 + j) % tiles_per_slot) * kTileKV;
        const int valid = min(kTileKV, p.L_slot - t0);
        if (!mbar_wait(s_full(g), cnt & 1u, abort_flag, p.dev_status, 600)) {
          ok = false;
          break;
        }
        __syncwarp();
        tc_fence_after_sync();
        // the whole row of S into registers, then hand the buffer back
        uint32_t v0[32], v1[32], v2[32], v3[32];
        tmem_ld_32x32(s_addr, v0);
        tmem_ld_32x32(s_addr + 32, v1);
        tmem_ld_32x32(s_addr + 64, v2);
        tmem_ld_32x32(s_addr + 96, v3);
        tmem_ld_wait();
        tc_fence_before_sync();
        mbar_arrive(s_free(g));
        // row maximum over the valid columns
        float m_tile;
        if (valid == kTileKV) {
          float ma = -INFINITY, mb = -INFINITY, mc = -INFINITY, md = -INFINITY;
#pragma unroll
          for (int i = 0; i < 32; i += 2) {
            ma = max3(ma, __uint_as_float(v0[i]), __uint_as_float(v0[i + 1]));
            mb = max3(mb, __uint_as_float(v1[i]), __uint_as_float(v1[i + 1]));
            mc = max3(mc, __uint_as_float(v2[i]), __uint_as_float(v2[i + 1]));
            md = max3(md, __uint_as_float(v3[i]), __uint_as_float(v3[i + 1]));
          }
          m_tile = fmaxf(fmaxf(ma, mb), fmaxf(mc, md));
        } else {
          m_tile = fmaxf(fmaxf(ragged_chunk_max(v0, valid), ragged_chunk_max(v1, valid - 32)),
                         fmaxf(ragged_chunk_max(v2, valid - 64), ragged_chunk_max(v3, valid - 96)));
        }
        const float m_new = fmaxf(m_run, m_tile * sc);
        float alpha = 1.f;
        if (j == 0) {
          m_run = m_new;  // O and L start from zero: nothing to rescale
        } else if (m_new > m_run + kRaise) {
          alpha = fast_exp2(m_run - m_new);
          m_run = m_new;
        }
        const bool rescale = __any_sync(0xffffffffu, alpha != 1.f);
        // P = exp2(S*scale - m) in fp32, summed in fp32, packed to fp16 for the tensor core:
        // pa = columns [0,64), pb = columns [64,128), two per 32-bit word
        uint32_t pa[32], pb[32];
        float sum0 = 0.f, sum1 = 0.f, sum2 = 0.f, sum3 = 0.f;
        if (valid == kTileKV) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float a0 = fast_exp2(fmaf(__uint_as_float(v0[2 * i]), sc, -m_run)), a1 = fast_exp2(fmaf(__uint_as_float(v0[2 * i + 1]), sc, -m_run));
            const float b0 = fast_exp2(fmaf(__uint_as_float(v1[2 * i]), sc, -m_run)), b1 = fast_exp2(fmaf(__uint_as_float(v1[2 * i + 1]), sc, -m_run));
            const float c0 = fast_exp2(fmaf(__uint_as_float(v2[2 * i]), sc, -m_run)), c1 = fast_exp2(fmaf(__uint_as_float(v2[2 * i + 1]), sc, -m_run));
            const float d0 = fast_exp2(fmaf(__uint_as_float(v3[2 * i]), sc, -m_run)), d1 = fast_exp2(fmaf(__uint_as_float(v3[2 * i + 1]), sc, -m_run));
            sum0 += a0 + a1, sum1 += b0 + b1, sum2 += c0 + c1, sum3 += d0 + d1;
            pa[i] = pack_f16x2(a0, a1), pa[16 + i] = pack_f16x2(b0, b1), pb[i] = pack_f16x2(c0, c1), pb[16 + i] = pack_f16x2(d0, d1);
          }
        } else {
          // ragged last tile of a slot: columns >= valid contribute nothing
          sum0 = ragged_chunk_p<0>(v0, pa, valid, sc, m_run);
          sum1 = ragged_chunk_p<16>(v1, pa, valid - 32, sc, m_run);
          sum2 = ragged_chunk_p<0>(v2, pb, valid - 64, sc, m_run);
          sum3 = ragged_chunk_p<16>(v3, pb, valid - 96, sc, m_run);
        }
        l_run = fmaf(l_run, alpha, (sum0 + sum1) + (sum2 + sum3));
        // the previous P V product of this group must have finished: it read the P buffer, and O
        // is only touched between two products
        if (j == 0) {
          if (pend_w >= 0 && !emit_pending()) {
            ok = false;
            break;
          }
        } else {
          if (!mbar_wait(o_full(g), (cnt - 1) & 1u, abort_flag, p.dev_status, 601)) {
            ok = false;
            break;
          }
          __syncwarp();
          tc_fence_after_sync();
          if (rescale) {
            uint32_t o0[32], o1[32];
            tmem_ld_32x32(o_addr, o0);
            tmem_ld_32x32(o_addr + 32, o1);
            tmem_ld_wait();
#pragma unroll
            for (int i = 0; i < 32; ++i) {
              o0[i] = __float_as_uint(__uint_as_float(o0[i]) * alpha);
              o1[i] = __float_as_uint(__uint_as_float(o1[i]) * alpha);
            }
            tmem_st_32x32(o_addr, o0);
            tmem_st_32x32(o_addr + 32, o1);
          }
        }
        // publish P in tensor memory
        tmem_st_32x32(p_addr, pa);
        tmem_st_32x32(p_addr + 32, pb);
        tmem_st_wait();
        tc_fence_before_sync();
        mbar_arrive(p_full(g));
      }
      if (!ok) break;
      pend_w = w, pend_l = l_run, pend_m = m_run;
    }
    if (ok && pend_w >= 0) {
      if (S == 1) {
        emit_pending();
      } else if (mbar_wait(o_full(g), (cnt - 1) & 1u, abort_flag, p.dev_status, 602)) {
        // kv_split > 1: keep the partial result for the merge
        __syncwarp();
        tc_fence_after_sync();
        uint32_t o0[32], o1[32];
        tmem_ld_32x32(o_addr, o0);
        tmem_ld_32x32(o_addr + 32, o1);
        tmem_ld_wait();
#pragma unroll
        for (int i = 0; i < 32; ++i) fin_o[i] = o0[i], fin_o[32 + i] = o1[i];
        fin_l = pend_l;
        fin_m = pend_m;
        fin_valid = true;
      }
    }
    // ---- kv_split > 1: merge the partial results of the cluster and write the output -------
    // (the producer / MMA warps take part in the same three barriers in their own branch)
    tc_fence_before_sync();
    __syncthreads();
    if (S > 1) {
      const int w = first_unit;
      const int n_groups = unit_groups(w);
      const bool softmax_thread = (warp < 8) && ((warp >> 2) < n_groups);
      const int sg = warp >> 2, srow = (warp & 3) * 32 + lane;     // group and row of a softmax thread
      const int grow = sg * kTileQ + srow;                                 // row within the unit's 256 queries
      // every CTA of the cluster has left its K/V loop: the K/V ring of each CTA is free and serves
      // as the receive buffer  [sender][66 values][rows owned] (fp32)
      cluster_sync_all();
      const int rows_owned = 2 * kTileQ / S;
      const uint32_t owner = softmax_thread ? static_cast<uint32_t>(grow / rows_owned) : 0u;
      const int lrow = grow % rows_owned;
      const uint32_t recv = smem_base + AttnSmem::kK;
      if (softmax_thread && owner != crank && fin_valid) {
        const uint32_t slot = (crank < owner) ? crank : crank - 1;
        const uint32_t base = map_to_cta(recv + ((slot * 66u) * rows_owned + lrow) * 4u, owner);
        const uint32_t stride = rows_owned * 4u;
  #pragma unroll
        for (int i = 0; i < kHeadDim; ++i) st_cluster_f32(base + i * stride, __uint_as_float(fin_o[i]));
        st_cluster_f32(base + 64u * stride, fin_l);
        st_cluster_f32(base + 65u * stride, fin_m);
      }
      cluster_sync_all();  // all partials have landed
      if (softmax_thread && owner == crank && fin_valid) {
        const float* rbuf = reinterpret_cast<const float*>(smem_gen + AttnSmem::kK);
        float m_all = fin_m;
        for (int s2 = 0; s2 < S - 1; ++s2) m_all = fmaxf(m_all, rbuf[(s2 * 66 + 65) * rows_owned + lrow]);
        const float own_scale = fast_exp2(fin_m - m_all);
        float l_all = fin_l * own_scale;
        float acc[kHeadDim];
  #pragma unroll
        for (int i = 0; i < kHeadDim; ++i) acc[i] = __uint_as_float(fin_o[i]) * own_scale;
        for (int s2 = 0; s2 < S - 1; ++s2) {
          const float* rb = rbuf + (s2 * 66) * rows_owned + lrow;
          const float sc2 = fast_exp2(rb[65 * rows_owned] - m_all);
          l_all = fmaf(rb[64 * rows_owned], sc2, l_all);
  #pragma unroll
          for (int i = 0; i < kHeadDim; ++i) acc[i] = fmaf(rb[i * rows_owned], sc2, acc[i]);
        }
        const int q_row = unit_q_row0(w) + grow;
        if (q_row < p.L_q) {
          const float inv_l = 1.f / l_all;
          __half* dst = p.out + (long long)unit_img(w) * p.out_img_stride + (long long)q_row * p.ld_out + unit_head(w) * kHeadDim;
  #pragma unroll
          for (int q = 0; q < 8; ++q) {
            uint4 u;
            u.x = pack_f16x2(acc[q * 8] * inv_l, acc[q * 8 + 1] * inv_l);
            u.y = pack_f16x2(acc[q * 8 + 2] * inv_l, acc[q * 8 + 3] * inv_l);
            u.z = pack_f16x2(acc[q * 8 + 4] * inv_l, acc[q * 8 + 5] * inv_l);
            u.w = pack_f16x2(acc[q * 8 + 6] * inv_l, acc[q * 8 + 7] * inv_l);
            *reinterpret_cast<uint4*>(dst + q * 8) = u;
          }
        }
      }
    }
  }
  // ---- teardown ---------------------------------------------------------------
  tc_fence_before_sync();
  __syncthreads();
  if (*abort_flag) {
    const unsigned long long t0 = global_timer_ns();
    while (global_timer_ns() - t0 < 200000ull) __nanosleep(1000);
    __syncthreads();
  }
  if (warp == 9) {
    __syncwarp();
    tc_fence_after_sync();
    tmem_dealloc(tmem_base, kTmemCols);
  }
}

static int g_force_attn_split = 0;  // test hook: 0 = choose
static int g_attn_tail_split = 1;   // serve an under-filled last round as half units (BXL_ATTN_TAIL_SPLIT=0 turns it off)

}  // namespace bxl

using namespace bxl;

extern "C" int bxl_debug_force_attn_split(int split) {
  if (split != 0 && split != 1 && split != 2 && split != 4) return fail(kErrInvalidArg, "bxl_debug_force_attn_split: 0, 1, 2 or 4");
  g_force_attn_split = split;
  return kOk;
}

extern "C" int bxl_attn_fwd_f16(const void* q, long long q_img_stride, long long ld_q, const void* const* kv_slots,
                                int n_slots, long long kv_img_stride, long long ld_kv, int v_col0, void* out,
                                long long out_img_stride, long long ld_out, int B, int heads, int L_q, int L_slot,
                                float scale, void* stream) {
  if (!q || !kv_slots || !out) return fail(kErrInvalidArg, "bxl_attn_fwd_f16: null pointer");
  if (n_slots < 1 || n_slots > kMaxSlots) return fail(kErrInvalidArg, "bxl_attn_fwd_f16: n_slots=%d (1..%d)", n_slots, kMaxSlots);
  if (B <= 0 || heads <= 0 || L_q <= 0 || L_slot <= 0) return fail(kErrInvalidArg, "bxl_attn_fwd_f16: non-positive extent");
  if (ld_q % 8 || ld_kv % 8 || ld_out % 8 || q_img_stride % 8 || kv_img_stride % 8 || out_img_stride % 8 || v_col0 % 8)
    return fail(kErrInvalidArg, "bxl_attn_fwd_f16: strides must be multiples of 8 elements");
  if (ld_q < heads * kHeadDim || ld_out < heads * kHeadDim || ld_kv < v_col0 + heads * kHeadDim || v_col0 < heads * kHeadDim)
    return fail(kErrInvalidArg, "bxl_attn_fwd_f16: row strides too small for %d heads of 64", heads);
  if ((reinterpret_cast<uintptr_t>(q) & 15u) || (reinterpret_cast<uintptr_t>(out) & 15u))
    return fail(kErrInvalidArg, "bxl_attn_fwd_f16: q/out must be 16-byte aligned");
  int* st = device_status_ptr();
  if (!st) return fail(kErrCuda, "bxl_attn_fwd_f16: no device status word");
  AttnParams p;
  memset(&p, 0, sizeof(p));
  {
    uint64_t dims[3] = {(uint64_t)(heads * kHeadDim), (uint64_t)L_q, (uint64_t)B};
    uint64_t str[2] = {(uint64_t)ld_q * 2, (uint64_t)q_img_stride * 2};
    uint32_t box[3] = {kHeadDim, kTileQ, 1};
    if (int rc = encode_tmap_f16(&p.q_map, q, 3, dims, str, box)) return rc;
  }
  for (int s = 0; s < kMaxSlots; ++s) {
    const void* base = kv_slots[s < n_slots ? s : 0];
    if (!base) return fail(kErrInvalidArg, "bxl_attn_fwd_f16: slot %d null", s);
    uint64_t dims[3] = {(uint64_t)(v_col0 + heads * kHeadDim), (uint64_t)L_slot, (uint64_t)B};
    uint64_t str[2] = {(uint64_t)ld_kv * 2, (uint64_t)kv_img_stride * 2};
    uint32_t box[3] = {kHeadDim, kTileKV, 1};
    if (int rc = encode_tmap_f16(&p.kv_map[s], base, 3, dims, str, box)) return rc;
  }
  p.n_slots = n_slots, p.L_q = L_q, p.L_slot = L_slot, p.heads = heads, p.B = B, p.v_col0 = v_col0;
  p.out = static_cast<__half*>(out);
  p.out_img_stride = out_img_stride, p.ld_out = ld_out;
  p.scale_log2e = scale * 1.4426950408889634f;
  p.dev_status = st;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (int rc = check_cuda(cudaFuncSetAttribute(attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, AttnSmem::kTotal),
                            "cudaFuncSetAttribute(attention)"))
      return rc;
    configured[dev] = true;
  }
  const int q_pairs = (L_q + 2 * kTileQ - 1) / (2 * kTileQ);
  const int work = q_pairs * heads * B;
  const int total_tiles = n_slots * ((L_slot + kTileKV - 1) / kTileKV);
  // K/V split: fewest rounds x tiles per round.  Without a split a CTA walks several units and
  // pays ~1 tile of bubble per unit plus ~2.5 once; with a split each cluster serves one unit and
  // pays ~2.5 tiles of set-up and ~1.5 for the merge.
  int split = 1;
  double best = 1e30;
  for (int s2 = 1; s2 <= 4; s2 *= 2) {
    if (s2 > total_tiles || (g_force_attn_split && s2 != g_force_attn_split)) continue;
    const int clusters = sm_count() / s2;
    const int rounds = (work + clusters - 1) / clusters;
    const double cost = (s2 == 1) ? rounds * (total_tiles + 1.0) + 2.5 : rounds * ((total_tiles + s2 - 1) / s2 + 2.5 + 1.5);
    if (cost < best - 1e-9) best = cost, split = s2;
  }
  p.kv_split = split;
  // A persistent grid whose last round would keep at most half of the SMs busy serves that round's
  // units as half units (one query tile each): twice the CTAs, about half the time.
  p.n_full = work;
  static int tail_env = -1;
  if (tail_env < 0) {
    const char* e = getenv("BXL_ATTN_TAIL_SPLIT");
    tail_env = (e && e[0] == '0') ? 0 : 1;
  }
  if (split == 1 && g_attn_tail_split && tail_env && L_q % (2 * kTileQ) == 0 && work > sm_count()) {
    const int rem = work % sm_count();
    if (rem > 0 && 2 * rem <= sm_count()) p.n_full = work - rem;
  }
  const int units = p.n_full + 2 * (work - p.n_full);
  const int grid = (split == 1) ? (units < sm_count() ? units : sm_count()) : work * split;
  return launch_kernel("attention_kernel launch", attention_kernel, dim3(grid), dim3(kAttnThreads), AttnSmem::kTotal,
                       (cudaStream_t)stream, split, p);
}
