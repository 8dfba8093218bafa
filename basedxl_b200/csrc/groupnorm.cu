// GroupNorm on an NHWC H-strip with cross-strip (possibly stale) moments, fused
// with the SiLU that follows it in the residual blocks.
//
//   pass 1  groupnorm_stats_kernel: per-(image, group) first and second raw
//           moments of the local strip, fp32.  Every CTA reduces a slab of
//           pixels; per-CTA partials go to scratch, and the last CTA to finish
//           (a self-resetting ticket counter in scratch) folds them, in fixed
//           order, into the moments buffer the strip publishes to its peers.
//   pass 2  groupnorm_apply_kernel: combines the fresh moments with the peers'
//           buffers (sync: average of all; stale: average of the stale buffers
//           plus the own fresh-minus-stale correction), forms the variance with
//           the negative-variance fallback and the local-count Bessel factor,
//           and writes y = (x - mean) * rstd * gamma + beta, optionally
//           y * sigmoid(y).
//
// Roofline: HBM.  Algorithmic bytes = read x + write y (2 * numel * 2 B); pass 1
// re-reads x, which for the strip sizes of this workload is served by L2.
#include "bxl_common.cuh"
#include "bxl_host.h"
#include "../../include/basedxl_b200.h"

namespace bxl {

constexpr int kGnMaxParts = 128;   // per-image partial slabs
constexpr int kGnMaxGroups = 64;
constexpr int kGnMaxC = 4096;

__device__ __forceinline__ void accumulate8(const uint4 u, float (&s1)[8], float (&s2)[8]) {
  const __half2 h[4] = {*reinterpret_cast<const __half2*>(&u.x), *reinterpret_cast<const __half2*>(&u.y),
                        *reinterpret_cast<const __half2*>(&u.z), *reinterpret_cast<const __half2*>(&u.w)};
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    const float2 f = __half22float2(h[j]);
    s1[2 * j] += f.x, s2[2 * j] = fmaf(f.x, f.x, s2[2 * j]);
    s1[2 * j + 1] += f.y, s2[2 * j + 1] = fmaf(f.y, f.y, s2[2 * j + 1]);
  }
}

// scratch layout: [0] ticket counter (int, kept at 0 between launches), then
// partials [B][parts][G][2] floats starting at byte 256
__global__ void __launch_bounds__(512) groupnorm_stats_kernel(const __half* __restrict__ x, long long img_stride, int HW,
                                                              int C, int G, int parts, float* __restrict__ partials,
                                                              int* __restrict__ ticket, float* __restrict__ moments, int B) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float s_part[];  // [rows][2][C]: every thread's channel sums / sums of squares, no atomics
  __shared__ int s_last;
  const int vecs = C / 8;               // 16-byte vectors per pixel
  const int rows = blockDim.x / vecs;   // pixels handled per sweep
  const int part = blockIdx.x, img = blockIdx.y;
  const int v = threadIdx.x % vecs, r = threadIdx.x / vecs;
  float s1[8], s2[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s1[j] = s2[j] = 0.f;
  if (r < rows) {
    const int per = (HW + parts - 1) / parts;
    const int p0 = part * per, p1 = min(HW, p0 + per);
    const __half* base = x + (long long)img * img_stride + (long long)v * 8;
    auto accumulate = [&](const uint4 u) { accumulate8(u, s1, s2); };
    int pix = p0 + r;
    // four pixels per trip: four independent 16-byte loads in flight per thread
    for (; pix + 3 * rows < p1; pix += 4 * rows) {
      const uint4 u0 = __ldg(reinterpret_cast<const uint4*>(base + (long long)pix * C));
      const uint4 u1 = __ldg(reinterpret_cast<const uint4*>(base + (long long)(pix + rows) * C));
      const uint4 u2 = __ldg(reinterpret_cast<const uint4*>(base + (long long)(pix + 2 * rows) * C));
      const uint4 u3 = __ldg(reinterpret_cast<const uint4*>(base + (long long)(pix + 3 * rows) * C));
      accumulate(u0), accumulate(u1), accumulate(u2), accumulate(u3);
    }
    for (; pix < p1; pix += rows) accumulate(__ldg(reinterpret_cast<const uint4*>(base + (long long)pix * C)));
    float* d1 = s_part + ((long long)r * 2) * C + v * 8;
    float* d2 = d1 + C;
    *reinterpret_cast<float4*>(d1) = make_float4(s1[0], s1[1], s1[2], s1[3]);
    *reinterpret_cast<float4*>(d1 + 4) = make_float4(s1[4], s1[5], s1[6], s1[7]);
    *reinterpret_cast<float4*>(d2) = make_float4(s2[0], s2[1], s2[2], s2[3]);
    *reinterpret_cast<float4*>(d2 + 4) = make_float4(s2[4], s2[5], s2[6], s2[7]);
  }
  __syncthreads();
  // one warp per (group, moment): lanes stride over the rows x channels-of-the-group sums, then a
  // shuffle tree - a fixed summation order, so the result does not depend on scheduling
  const int cpg = C / G;
  {
    const int lane_ = threadIdx.x & 31, warp_ = threadIdx.x >> 5, warps_ = blockDim.x >> 5;
    if (warp_ < warps_) {
      for (int i = warp_; i < 2 * G; i += warps_) {
        const int g = i % G, which = i / G;
        float acc = 0.f;
        for (int e = lane_; e < rows * cpg; e += 32) {
          const int rr = e / cpg, c = e - rr * cpg;
          acc += s_part[((long long)rr * 2 + which) * C + g * cpg + c];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane_ == 0) partials[(((long long)img * parts + part) * G + g) * 2 + which] = acc;
      }
    }
  }
  // last CTA of the whole grid folds the partials
  __threadfence();
  __syncthreads();
  if (threadIdx.x == 0) {
    const int total = gridDim.x * gridDim.y;
    const int t = atomicAdd(ticket, 1);
    s_last = (t == total - 1);
    if (s_last) *ticket = 0;  // ready for the next launch on this stream
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  // fold the partials: one warp per (image, group, moment), lanes striding over the slabs so
  // that the loads are independent; fixed summation order (lane-strided, then a shuffle tree)
  const float inv_n = 1.f / (float)((long long)cpg * HW);
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;
  if (warp >= warps) return;  // a trailing partial warp takes no part in the warp-wide shuffles
  for (int i = warp; i < B * G * 2; i += warps) {
    const int which = i % 2, g = (i / 2) % G, b = i / (2 * G);
    float acc = 0.f;
    for (int q = lane; q < parts; q += 32) acc += __ldcg(&partials[(((long long)b * parts + q) * G + g) * 2 + which]);
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
    // published layout [2][B][G]: first moments, then second moments
    if (lane == 0) moments[((long long)which * B + b) * G + g] = acc * inv_n;
  }
}

__device__ __forceinline__ float fast_tanh(float x) {
  float y;
  asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

struct GnPeers {
  const float* ptr[8];
};

// mode: 0 local, 1 sync (average of peers; own slot already holds the fresh moments),
//       2 stale (average of peers + fresh - peers[own])
__global__ void __launch_bounds__(512) groupnorm_apply_kernel(const __half* __restrict__ x, __half* __restrict__ y,
                                                              long long img_stride, int HW, int C, int G, int B,
                                                              const float* __restrict__ fresh, GnPeers peers, int n_peers,
                                                              int own, int mode, float eps, const __half* __restrict__ gamma,
                                                              const __half* __restrict__ beta, int silu, int parts) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float s_ab[];  // [2][C]: scale, shift per channel
  __shared__ float s_mean[kGnMaxGroups], s_rstd[kGnMaxGroups];
  const int img = blockIdx.y;
  const int cpg = C / G;
  if (threadIdx.x < G) {
    const int g = threadIdx.x;
    const long long i1 = (long long)img * G + g, i2 = ((long long)B + img) * G + g;
    const float f1 = fresh[i1], f2 = fresh[i2];
    float m1 = f1, m2 = f2;
    if (mode != 0 && n_peers > 0) {
      float a1 = 0.f, a2 = 0.f;
      for (int j = 0; j < n_peers; ++j) {
        a1 += (mode == 1 && j == own) ? f1 : peers.ptr[j][i1];
        a2 += (mode == 1 && j == own) ? f2 : peers.ptr[j][i2];
      }
      const float inv = 1.f / (float)n_peers;
      m1 = a1 * inv, m2 = a2 * inv;
      if (mode == 2) {
        m1 += f1 - peers.ptr[own][i1];
        m2 += f2 - peers.ptr[own][i2];
      }
    }
    float var = m2 - m1 * m1;
    if (var < 0.f) var = f2 - f1 * f1;
    const float n = (float)((long long)cpg * HW);
    var *= n / (n - 1.f);
    s_mean[g] = m1;
    s_rstd[g] = rsqrtf(var + eps);
  }
  __syncthreads();
  for (int c = threadIdx.x; c < C; c += blockDim.x) {
    const int g = c / cpg;
    const float ga = gamma ? __half2float(gamma[c]) : 1.f;
    const float be = beta ? __half2float(beta[c]) : 0.f;
    const float a = s_rstd[g] * ga;
    s_ab[c] = a;
    s_ab[C + c] = be - s_mean[g] * a;
  }
  __syncthreads();
  const int vecs = C / 8;
  const int rows = blockDim.x / vecs;
  const int v = threadIdx.x % vecs, r = threadIdx.x / vecs;
  if (r >= rows) return;
  float a[8], b[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = s_ab[v * 8 + j], b[j] = s_ab[C + v * 8 + j];
  const int per = (HW + parts - 1) / parts;
  const int p0 = blockIdx.x * per, p1 = min(HW, p0 + per);
  const long long off = (long long)img * img_stride + (long long)v * 8;
  for (int pix = p0 + r; pix < p1; pix += rows) {
    const uint4 u = *reinterpret_cast<const uint4*>(x + off + (long long)pix * C);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(h[j]);
      float y0 = f.x * a[2 * j] + b[2 * j];
      float y1 = f.y * a[2 * j + 1] + b[2 * j + 1];
      if (silu) {
        // y * sigmoid(y) with sigmoid(y) = 0.5 * tanh(0.5 y) + 0.5: one special-function op per value
        y0 = y0 * fmaf(0.5f, fast_tanh(0.5f * y0), 0.5f);
        y1 = y1 * fmaf(0.5f, fast_tanh(0.5f * y1), 0.5f);
      }
      oh[j] = __floats2half2_rn(y0, y1);
    }
    *reinterpret_cast<uint4*>(y + off + (long long)pix * C) = o;
  }
}

// ---- one-launch GroupNorm (local or stale moments) ------------------------------------
// A thread-block cluster owns one (image, channel block); a channel block is the smallest run of
// whole groups that is also a whole number of 16-byte vectors.  Each CTA of the cluster takes a
// range of pixels: it reads its slab ONCE (keeping it in shared memory when it fits), reduces
// the per-group sums, hands them to every CTA of the cluster through distributed shared
// memory, and after one cluster barrier normalises its slab from shared memory.  The moments
// the strip publishes are written by the cluster's first CTA, straight into the staging range
// when the caller passes it; the strip's first and last pixel rows (what a following 3x3
// convolution publishes to the neighbouring strips) can be written out on the way.
constexpr int kGnfMaxGroupsPerBlock = 8;
constexpr int kGnfMaxCluster = 8;

struct GnFusedParams {
  const __half* x;
  __half* y;
  long long img_stride;
  int HW, C, G, B;
  int cb;              // channels per block (multiple of 8 and of C / G)
  int cs;              // CTAs per cluster (pixel ranges)
  int keep;            // slab kept in shared memory between the two passes
  float* fresh_out;    // [2][B][G] moments of this strip, or null
  GnPeers peers;       // stale moments of every strip (mode 2)
  int n_peers, own, mode;  // mode 0: local, 2: stale
  float eps;
  const __half* gamma;
  const __half* beta;
  int silu;
  __half* halo_out;    // [2][B][W][C]: first and last pixel row of the strip's OUTPUT, or null
  int W;
};

__global__ void __launch_bounds__(512) groupnorm_fused_kernel(const GnFusedParams p) {
  pdl_launch_dependents();
  extern __shared__ __align__(16) unsigned char gnf_smem[];
  const int cb = p.cb, bv = cb / 8, cpg = p.C / p.G, gb = cb / cpg;
  const int rows = blockDim.x / bv;                       // pixels per sweep
  const uint32_t crank = p.cs > 1 ? cluster_ctarank() : 0u;
  const int cblk = blockIdx.x / p.cs, img = blockIdx.y;
  const int per = (p.HW + p.cs - 1) / p.cs;
  const int p0 = min(p.HW, (int)crank * per), p1 = min(p.HW, p0 + per);
  // shared-memory layout: exchange slots | per-group results | per-channel scale/shift | per-thread partials | slab
  float* s_xch = reinterpret_cast<float*>(gnf_smem);                       // [cs][gb][2]
  float* s_stat = s_xch + kGnfMaxCluster * kGnfMaxGroupsPerBlock * 2;      // [gb][2] mean, rstd; then stale terms [gb][4]
  float* s_ab = s_stat + kGnfMaxGroupsPerBlock * 6;                        // [2][cb]
  float* s_part = s_ab + 2 * cb;                                           // [rows][2][cb]
  uint4* s_slab = reinterpret_cast<uint4*>(s_part + (size_t)rows * 2 * cb + 2 * kGnfMaxGroupsPerBlock * 16);  // after the per-warp sums; [p1 - p0][bv] when kept
  const int v = threadIdx.x % bv, r = threadIdx.x / bv;
  const int g0 = cblk * gb;                               // first group of this block
  pdl_wait();
  // stale terms of this block's groups, read BEFORE any CTA publishes fresh moments into the
  // same buffer: avg over the strips' stale moments and the own stale moments
  if (p.mode == 2 && threadIdx.x < gb) {
    const int g = g0 + threadIdx.x;
    const long long i1 = (long long)img * p.G + g, i2 = ((long long)p.B + img) * p.G + g;
    float a1 = 0.f, a2 = 0.f;
    for (int j = 0; j < p.n_peers; ++j) a1 += p.peers.ptr[j][i1], a2 += p.peers.ptr[j][i2];
    const float inv = 1.f / (float)p.n_peers;
    float* t = s_stat + kGnfMaxGroupsPerBlock * 2 + threadIdx.x * 4;
    t[0] = a1 * inv, t[1] = a2 * inv, t[2] = p.peers.ptr[p.own][i1], t[3] = p.peers.ptr[p.own][i2];
  }
  // ---- pass 1: read the slab, per-thread channel sums
  float s1[8], s2[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) s1[j] = s2[j] = 0.f;
  const __half* xb = p.x + (long long)img * p.img_stride + (long long)cblk * cb + (long long)v * 8;
  if (r < rows) {
    int pix = p0 + r;
    for (; pix + 3 * rows < p1; pix += 4 * rows) {
      const uint4 u0 = __ldg(reinterpret_cast<const uint4*>(xb + (long long)pix * p.C));
      const uint4 u1 = __ldg(reinterpret_cast<const uint4*>(xb + (long long)(pix + rows) * p.C));
      const uint4 u2 = __ldg(reinterpret_cast<const uint4*>(xb + (long long)(pix + 2 * rows) * p.C));
      const uint4 u3 = __ldg(reinterpret_cast<const uint4*>(xb + (long long)(pix + 3 * rows) * p.C));
      if (p.keep) {
        s_slab[(size_t)(pix - p0) * bv + v] = u0, s_slab[(size_t)(pix + rows - p0) * bv + v] = u1;
        s_slab[(size_t)(pix + 2 * rows - p0) * bv + v] = u2, s_slab[(size_t)(pix + 3 * rows - p0) * bv + v] = u3;
      }
      accumulate8(u0, s1, s2), accumulate8(u1, s1, s2), accumulate8(u2, s1, s2), accumulate8(u3, s1, s2);
    }
    for (; pix < p1; pix += rows) {
      const uint4 u = __ldg(reinterpret_cast<const uint4*>(xb + (long long)pix * p.C));
      if (p.keep) s_slab[(size_t)(pix - p0) * bv + v] = u;
      accumulate8(u, s1, s2);
    }
    float* d1 = s_part + ((size_t)r * 2) * cb + v * 8;
    float* d2 = d1 + cb;
    *reinterpret_cast<float4*>(d1) = make_float4(s1[0], s1[1], s1[2], s1[3]);
    *reinterpret_cast<float4*>(d1 + 4) = make_float4(s1[4], s1[5], s1[6], s1[7]);
    *reinterpret_cast<float4*>(d2) = make_float4(s2[0], s2[1], s2[2], s2[3]);
    *reinterpret_cast<float4*>(d2 + 4) = make_float4(s2[4], s2[5], s2[6], s2[7]);
  }
  __syncthreads();
  // ---- this CTA's per-group sums, in a fixed order, sent to every CTA of the cluster.  Every warp
  //      folds its share of the pixel rows for every (group, moment); the per-warp results are then
  //      added in warp order: the summation order is fixed, whatever the scheduling.
  {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, warps = blockDim.x >> 5;  // whole warps only
    float* s_red = s_part + (size_t)rows * 2 * cb;   // [2 * gb][warps]; lives behind the per-thread partials (see the host's sizing)
    if (warp < warps) {
      const int rpw = (rows + warps - 1) / warps;    // pixel rows per warp
      const int r_lo = min(rows, warp * rpw), r_hi = min(rows, r_lo + rpw);
      for (int i = 0; i < 2 * gb; ++i) {
        const int g = i >> 1, which = i & 1;
        float acc = 0.f;
        for (int e = lane; e < (r_hi - r_lo) * cpg; e += 32) {
          const int rr = r_lo + e / cpg, c = e % cpg;
          acc += s_part[((size_t)rr * 2 + which) * cb + g * cpg + c];
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
        if (lane == 0) s_red[i * warps + warp] = acc;
      }
    }
    __syncthreads();
    if (threadIdx.x < 2 * gb * p.cs) {
      const int i = threadIdx.x % (2 * gb), dst_cta = threadIdx.x / (2 * gb);
      float acc = 0.f;
      for (int w = 0; w < warps; ++w) acc += s_red[i * warps + w];
      const int g = i >> 1, which = i & 1;
      const uint32_t dst = smem_u32(&s_xch[((int)crank * kGnfMaxGroupsPerBlock + g) * 2 + which]);
      if (p.cs > 1) st_cluster_f32(map_to_cta(dst, (uint32_t)dst_cta), acc);
      else s_xch[g * 2 + which] = acc;
    }
  }
  if (p.cs > 1) cluster_sync_all();
  else __syncthreads();
  // ---- moments of the block's groups; combination with the stale moments; scale / shift
  if (threadIdx.x < gb) {
    const int g = threadIdx.x;
    float a1 = 0.f, a2 = 0.f;
    for (int j = 0; j < p.cs; ++j) a1 += s_xch[(j * kGnfMaxGroupsPerBlock + g) * 2], a2 += s_xch[(j * kGnfMaxGroupsPerBlock + g) * 2 + 1];
    const float n = (float)((long long)cpg * p.HW);
    const float f1 = a1 / n, f2 = a2 / n;
    float m1 = f1, m2 = f2;
    if (p.mode == 2) {
      const float* t = s_stat + kGnfMaxGroupsPerBlock * 2 + g * 4;
      m1 = t[0] + (f1 - t[2]);
      m2 = t[1] + (f2 - t[3]);
    }
    float var = m2 - m1 * m1;
    if (var < 0.f) var = f2 - f1 * f1;
    var *= n / (n - 1.f);
    s_stat[g * 2] = m1;
    s_stat[g * 2 + 1] = rsqrtf(var + p.eps);
    if (crank == 0 && p.fresh_out) {
      p.fresh_out[(long long)img * p.G + g0 + g] = f1;
      p.fresh_out[((long long)p.B + img) * p.G + g0 + g] = f2;
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < cb; c += blockDim.x) {
    const int g = c / cpg, ch = cblk * cb + c;
    const float ga = p.gamma ? __half2float(p.gamma[ch]) : 1.f;
    const float be = p.beta ? __half2float(p.beta[ch]) : 0.f;
    const float a = s_stat[g * 2 + 1] * ga;
    s_ab[c] = a;
    s_ab[cb + c] = be - s_stat[g * 2] * a;
  }
  __syncthreads();
  // ---- pass 2: normalise (+ SiLU) and store
  if (r >= rows) return;
  float a[8], b[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) a[j] = s_ab[v * 8 + j], b[j] = s_ab[cb + v * 8 + j];
  __half* yb = p.y + (long long)img * p.img_stride + (long long)cblk * cb + (long long)v * 8;
  const int last_row0 = p.HW - p.W;
  for (int pix = p0 + r; pix < p1; pix += rows) {
    const uint4 u = p.keep ? s_slab[(size_t)(pix - p0) * bv + v] : *reinterpret_cast<const uint4*>(xb + (long long)pix * p.C);
    const __half2* h = reinterpret_cast<const __half2*>(&u);
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 f = __half22float2(h[j]);
      float y0 = f.x * a[2 * j] + b[2 * j];
      float y1 = f.y * a[2 * j + 1] + b[2 * j + 1];
      if (p.silu) {
        y0 = y0 * fmaf(0.5f, fast_tanh(0.5f * y0), 0.5f);
        y1 = y1 * fmaf(0.5f, fast_tanh(0.5f * y1), 0.5f);
      }
      oh[j] = __floats2half2_rn(y0, y1);
    }
    *reinterpret_cast<uint4*>(yb + (long long)pix * p.C) = o;
    if (p.halo_out) {
      if (pix < p.W)
        *reinterpret_cast<uint4*>(p.halo_out + ((long long)img * p.W + pix) * p.C + (long long)cblk * cb + v * 8) = o;
      if (pix >= last_row0)
        *reinterpret_cast<uint4*>(p.halo_out + (((long long)p.B + img) * p.W + (pix - last_row0)) * p.C + (long long)cblk * cb + v * 8) = o;
    }
  }
}

static int gn_threads(int C) {
  const int vecs = C / 8;
  int k = 512 / vecs;
  if (k < 1) k = 1;
  return vecs * k;
}

// per-thread partial sums of the statistics kernel: [rows][2][C] floats (at most 32 KB)
static size_t gn_stats_smem(int C) { return (size_t)(gn_threads(C) / (C / 8)) * 2 * C * sizeof(float); }

static int gn_parts(int HW, int C, int B) {
  const int rows = gn_threads(C) / (C / 8);
  int parts = (HW + rows * 16 - 1) / (rows * 16);  // >= 16 pixels per thread: the per-CTA fold is amortised
  const int cap = max(1, (sm_count() * 2) / max(1, B));
  if (parts > cap) parts = cap;
  if (parts > kGnMaxParts) parts = kGnMaxParts;
  if (parts < 1) parts = 1;
  return parts;
}

static int gn_check(const char* who, const void* x, int B, int HW, int C, int G, long long img_stride) {
  if (!x) return fail(kErrInvalidArg, "%s: null input", who);
  if (B <= 0 || HW <= 0 || C <= 0 || G <= 0) return fail(kErrInvalidArg, "%s: non-positive extent", who);
  if (C % 8 || C % G) return fail(kErrUnsupported, "%s: C=%d must be a multiple of 8 and of the group count %d", who, C, G);
  if (C > kGnMaxC || G > kGnMaxGroups || C / 8 > 512) return fail(kErrTooLarge, "%s: C=%d / G=%d beyond the supported maximum", who, C, G);
  if (img_stride % 8 || (reinterpret_cast<uintptr_t>(x) & 15u)) return fail(kErrInvalidArg, "%s: x must be 16-byte aligned", who);
  return kOk;
}

}  // namespace bxl

using namespace bxl;

extern "C" long long bxl_groupnorm_scratch_bytes(int B, int G) {
  if (B <= 0 || G <= 0) return 0;
  return 256 + (long long)B * kGnMaxParts * G * 2 * sizeof(float);
}

extern "C" int bxl_groupnorm_stats_f16(const void* x, long long img_stride, int B, int HW, int C, int G, float* moments,
                                       void* scratch, long long scratch_bytes, void* stream) {
  if (int rc = gn_check("bxl_groupnorm_stats_f16", x, B, HW, C, G, img_stride)) return rc;
  if (!moments || !scratch) return fail(kErrInvalidArg, "bxl_groupnorm_stats_f16: null output/scratch");
  if (scratch_bytes < bxl_groupnorm_scratch_bytes(B, G)) return fail(kErrTooLarge, "bxl_groupnorm_stats_f16: scratch too small");
  const int threads = gn_threads(C), parts = gn_parts(HW, C, B);
  int* ticket = static_cast<int*>(scratch);
  float* partials = reinterpret_cast<float*>(static_cast<char*>(scratch) + 256);
  return launch_kernel("groupnorm_stats_kernel launch", groupnorm_stats_kernel, dim3(parts, B), dim3(threads), gn_stats_smem(C),
                       (cudaStream_t)stream, 1, static_cast<const __half*>(x), img_stride, HW, C, G, parts, partials, ticket,
                       moments, B);
}

extern "C" int bxl_groupnorm_apply_f16(const void* x, void* y, long long img_stride, int B, int HW, int C, int G,
                                       const float* fresh_moments, const float* const* peer_moments, int n_peers, int own,
                                       int mode, float eps, const void* gamma, const void* beta, int silu, void* stream) {
  if (int rc = gn_check("bxl_groupnorm_apply_f16", x, B, HW, C, G, img_stride)) return rc;
  if (!y || !fresh_moments) return fail(kErrInvalidArg, "bxl_groupnorm_apply_f16: null pointer");
  if (mode < 0 || mode > 2) return fail(kErrInvalidArg, "bxl_groupnorm_apply_f16: mode %d", mode);
  if (mode != 0 && (n_peers < 1 || n_peers > 8 || !peer_moments || own < 0 || own >= n_peers))
    return fail(kErrInvalidArg, "bxl_groupnorm_apply_f16: bad peer table (n=%d own=%d)", n_peers, own);
  GnPeers peers;
  for (int j = 0; j < 8; ++j) peers.ptr[j] = (mode != 0 && j < n_peers) ? peer_moments[j] : nullptr;
  if (mode != 0)
    for (int j = 0; j < n_peers; ++j)
      if (!peers.ptr[j] && !(mode == 1 && j == own)) return fail(kErrInvalidArg, "bxl_groupnorm_apply_f16: peer %d null", j);
  const int threads = gn_threads(C);
  const int rows = threads / (C / 8);
  int parts = (HW + rows * 2 - 1) / (rows * 2);
  const int cap = max(1, (sm_count() * 8) / B);
  if (parts > cap) parts = cap;
  if (parts < 1) parts = 1;
  return launch_kernel("groupnorm_apply_kernel launch", groupnorm_apply_kernel, dim3(parts, B), dim3(threads), 2 * C * sizeof(float),
                       (cudaStream_t)stream, 1, static_cast<const __half*>(x), static_cast<__half*>(y), img_stride, HW, C, G, B,
                       fresh_moments, peers, mode == 0 ? 0 : n_peers, own, mode, eps, static_cast<const __half*>(gamma),
                       static_cast<const __half*>(beta), silu, parts);
}

// Channel block of the one-launch kernel: whole groups and whole 16-byte vectors.
static int gnf_block_channels(int C, int G) {
  const int cpg = C / G;
  int cb = cpg;
  while (cb % 8) cb += cpg;
  return cb;
}

extern "C" int bxl_groupnorm_fused_f16(const void* x, void* y, long long img_stride, int B, int H, int W, int C, int G,
                                       float* fresh_out, const float* const* peer_moments, int n_peers, int own, int mode,
                                       float eps, const void* gamma, const void* beta, int silu, void* halo_out,
                                       void* stream) {
  const int HW = H * W;
  if (int rc = gn_check("bxl_groupnorm_fused_f16", x, B, HW, C, G, img_stride)) return rc;
  if (!y) return fail(kErrInvalidArg, "bxl_groupnorm_fused_f16: null output");
  if (mode != 0 && mode != 2) return fail(kErrInvalidArg, "bxl_groupnorm_fused_f16: mode %d (0 = local, 2 = stale; the synchronous mode needs the two-launch form)", mode);
  if (mode == 2 && (n_peers < 1 || n_peers > 8 || !peer_moments || own < 0 || own >= n_peers))
    return fail(kErrInvalidArg, "bxl_groupnorm_fused_f16: bad peer table (n=%d own=%d)", n_peers, own);
  const int cb = gnf_block_channels(C, G);
  if (C % cb || cb / (C / G) > kGnfMaxGroupsPerBlock || cb > 512)
    return fail(kErrUnsupported, "bxl_groupnorm_fused_f16: C=%d with %d groups does not split into channel blocks of whole groups and whole vectors", C, G);
  if (halo_out && (reinterpret_cast<uintptr_t>(halo_out) & 15u)) return fail(kErrInvalidArg, "bxl_groupnorm_fused_f16: halo_out must be 16-byte aligned");
  GnFusedParams p;
  memset(&p, 0, sizeof(p));
  for (int j = 0; j < 8; ++j) p.peers.ptr[j] = (mode == 2 && j < n_peers) ? peer_moments[j] : nullptr;
  if (mode == 2)
    for (int j = 0; j < n_peers; ++j)
      if (!p.peers.ptr[j]) return fail(kErrInvalidArg, "bxl_groupnorm_fused_f16: peer %d null", j);
  const int nblk = C / cb, bv = cb / 8;
  // pixel ranges per cluster: one CTA per SM or a little more (every further CTA costs a cluster
  // exchange and idles threads), slabs small enough to keep on chip
  int cs = 1;
  while (cs < kGnfMaxCluster && (long long)B * nblk * cs < sm_count() && HW / (cs * 2) >= 32) cs *= 2;
  while (cs < kGnfMaxCluster && (long long)HW * cb * 2 / cs > 160 * 1024) cs *= 2;
  const int per = (HW + cs - 1) / cs;
  const long long slab = (long long)per * cb * 2;
  // threads: one pixel row per thread row, at most 512 threads, whole warps, a whole number of pixel rows
  auto fixed_smem = [&](int th) {
    return (size_t)(kGnfMaxCluster * kGnfMaxGroupsPerBlock * 2 + kGnfMaxGroupsPerBlock * 6 + 2 * cb) * 4 + (size_t)(th / bv) * 2 * cb * 4 +
           (size_t)2 * kGnfMaxGroupsPerBlock * 16 * 4;
  };
  int rows_t = per < 512 / bv ? per : 512 / bv;
  if (slab + (long long)fixed_smem(rows_t * bv) > 200 * 1024 && rows_t > 256 / bv) rows_t = 256 / bv;
  if (rows_t < 1) rows_t = 1;
  // whole warps (the reductions run on whole warps) and enough threads for the cluster exchange
  int threads = ((rows_t * bv + 31) / 32) * 32;
  if (threads < 128) threads = 128;
  const int keep = slab + (long long)fixed_smem(threads) <= 200 * 1024;
  const size_t smem = fixed_smem(threads) + (keep ? (size_t)slab : 0) + 16;
  static bool configured[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev >= 0 && dev < 64 && !configured[dev]) {
    if (int rc = check_cuda(cudaFuncSetAttribute(groupnorm_fused_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 208 * 1024),
                            "cudaFuncSetAttribute(groupnorm_fused)"))
      return rc;
    configured[dev] = true;
  }
  p.x = static_cast<const __half*>(x), p.y = static_cast<__half*>(y), p.img_stride = img_stride;
  p.HW = HW, p.C = C, p.G = G, p.B = B, p.cb = cb, p.cs = cs, p.keep = keep;
  p.fresh_out = fresh_out, p.n_peers = mode == 2 ? n_peers : 0, p.own = own, p.mode = mode, p.eps = eps;
  p.gamma = static_cast<const __half*>(gamma), p.beta = static_cast<const __half*>(beta), p.silu = silu;
  p.halo_out = static_cast<__half*>(halo_out), p.W = W;
  return launch_kernel("groupnorm_fused_kernel launch", groupnorm_fused_kernel, dim3(cs * nblk, B), dim3(threads), smem,
                       (cudaStream_t)stream, cs, p);
}

// ---- statistics without caller-provided scratch ------------------------------------
// Some hosts of this library cannot hand it device memory at call time: an
// inference server that reserved its whole memory budget up front and forbids
// cudaMalloc inside operator callbacks (it may fail, and it synchronises the whole
// device), or a plugin invoked by a runtime that only passes input and output
// pointers.  For them the scratch of the statistics kernel lives in this
// file-scope device array, present once on every GPU that loads the library, for
// the life of the process.
namespace bxl {
constexpr int kGnStaticMaxBG = 256;  // largest images x groups product served
constexpr long long kGnStaticBytes = 256 + (long long)kGnStaticMaxBG * kGnMaxParts * 2 * sizeof(float);  // 262,400 B
static __device__ __align__(256) unsigned char g_gn_static_scratch[kGnStaticBytes];
// device address of the array, per device (the symbol itself is only a host-side handle)
static void* g_gn_static_ptr[64] = {};
}  // namespace bxl

extern "C" long long bxl_groupnorm_stats_noalloc_max_bg(void) { return kGnStaticMaxBG; }

extern "C" int bxl_groupnorm_stats_noalloc_f16(const void* x, long long img_stride, int B, int HW, int C, int G,
                                               float* moments, void* stream) {
  if (int rc = gn_check("bxl_groupnorm_stats_noalloc_f16", x, B, HW, C, G, img_stride)) return rc;
  if (!moments) return fail(kErrInvalidArg, "bxl_groupnorm_stats_noalloc_f16: null output");
  if ((long long)B * G > kGnStaticMaxBG)
    return fail(kErrTooLarge,
                "bxl_groupnorm_stats_noalloc_f16: B*G = %lld exceeds the built-in scratch (B*G <= %d); use "
                "bxl_groupnorm_stats_f16 with caller-owned scratch",
                (long long)B * G, kGnStaticMaxBG);
  int dev = 0;
  if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
  if (dev < 0 || dev >= 64) return fail(kErrUnsupported, "bxl_groupnorm_stats_noalloc_f16: device index %d", dev);
  if (!g_gn_static_ptr[dev]) {
    // first call on this device: resolve the array's device address (current device)
    void* ptr = nullptr;
    if (int rc = check_cuda(cudaGetSymbolAddress(&ptr, g_gn_static_scratch), "cudaGetSymbolAddress(static scratch)")) return rc;
    g_gn_static_ptr[dev] = ptr;
  }
  char* scratch = static_cast<char*>(g_gn_static_ptr[dev]);
  cudaStream_t s = (cudaStream_t)stream;
  // the ticket word must start at zero whatever an earlier call left behind
  if (int rc = check_cuda(cudaMemsetAsync(scratch, 0, 256, s), "clear ticket")) return rc;
  const int threads = gn_threads(C), parts = gn_parts(HW, C, B);
  groupnorm_stats_kernel<<<dim3(parts, B), threads, gn_stats_smem(C), s>>>(
      static_cast<const __half*>(x), img_stride, HW, C, G, parts, reinterpret_cast<float*>(scratch + 256),
      reinterpret_cast<int*>(scratch), moments, B);
  return check_cuda(cudaGetLastError(), "groupnorm_stats_kernel launch (static scratch)");
}

