// HBM-bound helpers around the tensor-core kernels, all on NHWC fp16:
// halo packing, the two direct 3x3 convolutions at the ends of the network
// (4 -> 320 and 320 -> 4 channels, too thin for tensor-core tiles), nearest 2x
// up-sampling, LayerNorm and GEGLU.
// Roofline for every kernel here: HBM; algorithmic bytes = inputs read once +
// outputs written once.
#include "bxl_common.cuh"
#include "bxl_host.h"
#include "../../include/basedxl_b200.h"

namespace bxl {

// ---- halo pack: first and last `pad` rows of a strip -> [2][B][pad][W][C] ----
__global__ void halo_pack_kernel(const uint4* __restrict__ x, long long img_stride_v, uint4* __restrict__ out, int B, int H,
                                 long long row_v, int pad) {
  pdl_launch_dependents();
  pdl_wait();
  const long long per = (long long)pad * row_v;  // vectors per (side, image)
  const long long total = 2ll * B * per;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long within = i % per;
    const int img = (i / per) % B;
    const int side = i / (per * B);
    const long long src_row0 = side == 0 ? 0 : (long long)(H - pad) * row_v;
    out[i] = x[(long long)img * img_stride_v + src_row0 + within];
  }
}

// ---- direct 3x3 conv, few input channels (conv_in) -----------------------------
// thread = (pixel, 8 output channels); weights [C_out][9][C_in] staged as fp32 in
// shared memory.
__global__ void conv3x3_small_cin_kernel(const __half* __restrict__ x, long long x_img_stride, const __half* __restrict__ top,
                                         const __half* __restrict__ bot, long long halo_img_stride,
                                         const __half* __restrict__ w, const __half* __restrict__ bias, __half* __restrict__ y,
                                         int B, int Cin, int Cout, int H, int W) {
  pdl_launch_dependents();
  pdl_wait();
  extern __shared__ float s_w[];  // [9*Cin][Cout]: threads of a warp (consecutive output vectors) read consecutive words
  const int K = 9 * Cin;
  for (int i = threadIdx.x; i < Cout * K; i += blockDim.x) s_w[(i % K) * Cout + i / K] = __half2float(w[i]);
  __syncthreads();
  const int ovecs = Cout / 8;
  const long long total = (long long)B * H * W * ovecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ov = i % ovecs;
    const long long pix = i / ovecs;
    const int ox = pix % W;
    const int oy = (pix / W) % H;
    const int img = pix / ((long long)W * H);
    float acc[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) acc[j] = bias ? __half2float(bias[ov * 8 + j]) : 0.f;
    for (int ky = 0; ky < 3; ++ky) {
      const int iy = oy + ky - 1;
      const __half* rowp;
      if (iy < 0) {
        if (!top) continue;
        rowp = top + (long long)img * halo_img_stride;
      } else if (iy >= H) {
        if (!bot) continue;
        rowp = bot + (long long)img * halo_img_stride;
      } else {
        rowp = x + (long long)img * x_img_stride + (long long)iy * W * Cin;
      }
      for (int kx = 0; kx < 3; ++kx) {
        const int ix = ox + kx - 1;
        if (ix < 0 || ix >= W) continue;
        const __half* px = rowp + (long long)ix * Cin;
        const int kbase = (ky * 3 + kx) * Cin;
        for (int c = 0; c < Cin; ++c) {
          const float v = __half2float(px[c]);
          const float4 w0 = *reinterpret_cast<const float4*>(&s_w[(kbase + c) * Cout + ov * 8]);
          const float4 w1 = *reinterpret_cast<const float4*>(&s_w[(kbase + c) * Cout + ov * 8 + 4]);
          acc[0] += v * w0.x, acc[1] += v * w0.y, acc[2] += v * w0.z, acc[3] += v * w0.w;
          acc[4] += v * w1.x, acc[5] += v * w1.y, acc[6] += v * w1.z, acc[7] += v * w1.w;
        }
      }
    }
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(acc[2 * j], acc[2 * j + 1]);
    *reinterpret_cast<uint4*>(y + pix * Cout + ov * 8) = o;
  }
}

// The same for C_in == 4 (the latent input of the UNet): a thread computes FOUR consecutive
// pixels of a row for its 8 output channels, so every weight vector fetched from shared memory
// serves four pixels (the one-pixel form above is bound by those fetches), and the 3 x 6 input
// pixels it needs are read once as 8-byte vectors.
__global__ void __launch_bounds__(256) conv3x3_cin4_kernel(const __half* __restrict__ x, long long x_img_stride,
                                                          const __half* __restrict__ top, const __half* __restrict__ bot,
                                                          long long halo_img_stride, const __half* __restrict__ w,
                                                          const __half* __restrict__ bias, __half* __restrict__ y, int B,
                                                          int Cout, int H, int W) {
  pdl_launch_dependents();
  pdl_wait();
  // weights as fp32, [36 taps x channels][2 halves][Cout / 8][4]: the threads of a warp (consecutive
  // output vectors) read consecutive 16-byte words, first the lower four channels, then the upper four
  extern __shared__ float s_w[];
  constexpr int K = 36;
  const int ovecs = Cout / 8;
  {
    // 16-byte loads, eight in flight per thread (one load per element made this loop, not the
    // convolution, the longest part of the kernel)
    const int nvec = Cout * K / 8;  // Cout is a multiple of 8
    const uint4* wv = reinterpret_cast<const uint4*>(w);
    for (int base = threadIdx.x; base < nvec; base += 8 * blockDim.x) {
      uint4 buf[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int vi = base + j * blockDim.x;
        buf[j] = vi < nvec ? wv[vi] : make_uint4(0u, 0u, 0u, 0u);
      }
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        const int vi = base + j * blockDim.x;
        if (vi >= nvec) continue;
        const __half* hv = reinterpret_cast<const __half*>(&buf[j]);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int i = vi * 8 + e;
          const int o = i / K, k = i % K;
          s_w[((k * 2 + ((o >> 2) & 1)) * ovecs + (o >> 3)) * 4 + (o & 3)] = __half2float(hv[e]);
        }
      }
    }
  }
  __syncthreads();
  const int wq = (W + 3) / 4;  // groups of four pixels per row
  const long long total = (long long)B * H * wq * ovecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int ov = i % ovecs;
    const long long grp = i / ovecs;
    const int ox0 = static_cast<int>(grp % wq) * 4;
    const int oy = static_cast<int>((grp / wq) % H);
    const int img = static_cast<int>(grp / ((long long)wq * H));
    float acc[4][8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float b = bias ? __half2float(bias[ov * 8 + j]) : 0.f;
#pragma unroll
      for (int q = 0; q < 4; ++q) acc[q][j] = b;
    }
#pragma unroll
    for (int ky = 0; ky < 3; ++ky) {
      const int iy = oy + ky - 1;
      const __half* rowp = nullptr;
      if (iy < 0) {
        if (top) rowp = top + (long long)img * halo_img_stride;
      } else if (iy >= H) {
        if (bot) rowp = bot + (long long)img * halo_img_stride;
      } else {
        rowp = x + (long long)img * x_img_stride + (long long)iy * W * 4;
      }
      if (!rowp) continue;
      float v[6][4];  // input pixels ox0-1 .. ox0+4, zero outside the row
#pragma unroll
      for (int t = 0; t < 6; ++t) {
        const int ix = ox0 + t - 1;
        uint2 u = make_uint2(0u, 0u);
        if (ix >= 0 && ix < W) u = *reinterpret_cast<const uint2*>(rowp + (long long)ix * 4);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x)), b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
        v[t][0] = a.x, v[t][1] = a.y, v[t][2] = b.x, v[t][3] = b.y;
      }
#pragma unroll
      for (int kx = 0; kx < 3; ++kx) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const float* wp = &s_w[((((ky * 3 + kx) * 4 + c) * 2) * ovecs + ov) * 4];
          const float4 w0 = *reinterpret_cast<const float4*>(wp), w1 = *reinterpret_cast<const float4*>(wp + ovecs * 4);
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float a = v[q + kx][c];
            acc[q][0] = fmaf(a, w0.x, acc[q][0]), acc[q][1] = fmaf(a, w0.y, acc[q][1]);
            acc[q][2] = fmaf(a, w0.z, acc[q][2]), acc[q][3] = fmaf(a, w0.w, acc[q][3]);
            acc[q][4] = fmaf(a, w1.x, acc[q][4]), acc[q][5] = fmaf(a, w1.y, acc[q][5]);
            acc[q][6] = fmaf(a, w1.z, acc[q][6]), acc[q][7] = fmaf(a, w1.w, acc[q][7]);
          }
        }
      }
    }
    const long long pix0 = ((long long)img * H + oy) * W + ox0;
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      if (ox0 + q >= W) break;
      uint4 o;
      __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
      for (int j = 0; j < 4; ++j) oh[j] = __floats2half2_rn(acc[q][2 * j], acc[q][2 * j + 1]);
      *reinterpret_cast<uint4*>(y + (pix0 + q) * Cout + ov * 8) = o;
    }
  }
}

// ---- direct 3x3 conv, few output channels (conv_out) ----------------------------
// one warp per output pixel; lanes stride over 16-byte input vectors of the 9 taps.
template <int COUT>
__global__ void conv3x3_small_cout_kernel(const __half* __restrict__ x, long long x_img_stride, const __half* __restrict__ top,
                                          const __half* __restrict__ bot, long long halo_img_stride,
                                          const __half* __restrict__ w, const __half* __restrict__ bias, __half* __restrict__ y,
                                          int B, int Cin, int H, int W) {
  pdl_launch_dependents();
  pdl_wait();
  const int warps_per_block = blockDim.x / 32;
  const int lane = threadIdx.x & 31;
  const long long total = (long long)B * H * W;
  const int vecs = Cin / 8;
  for (long long pix = blockIdx.x * (long long)warps_per_block + (threadIdx.x >> 5); pix < total;
       pix += (long long)gridDim.x * warps_per_block) {
    const int ox = pix % W;
    const int oy = (pix / W) % H;
    const int img = pix / ((long long)W * H);
    float acc[COUT];
#pragma unroll
    for (int j = 0; j < COUT; ++j) acc[j] = 0.f;
    for (int ky = 0; ky < 3; ++ky) {
      const int iy = oy + ky - 1;
      const __half* rowp;
      if (iy < 0) {
        if (!top) continue;
        rowp = top + (long long)img * halo_img_stride;
      } else if (iy >= H) {
        if (!bot) continue;
        rowp = bot + (long long)img * halo_img_stride;
      } else {
        rowp = x + (long long)img * x_img_stride + (long long)iy * W * Cin;
      }
      for (int kx = 0; kx < 3; ++kx) {
        const int ix = ox + kx - 1;
        if (ix < 0 || ix >= W) continue;
        const __half* px = rowp + (long long)ix * Cin;
        const int tap = ky * 3 + kx;
        for (int v = lane; v < vecs; v += 32) {
          const uint4 u = *reinterpret_cast<const uint4*>(px + v * 8);
          const __half2* xh = reinterpret_cast<const __half2*>(&u);
#pragma unroll
          for (int j = 0; j < COUT; ++j) {
            const uint4 wu = *reinterpret_cast<const uint4*>(w + ((long long)j * 9 + tap) * Cin + v * 8);
            const __half2* wh = reinterpret_cast<const __half2*>(&wu);
#pragma unroll
            for (int q = 0; q < 4; ++q) {
              const float2 a = __half22float2(xh[q]), b = __half22float2(wh[q]);
              acc[j] += a.x * b.x + a.y * b.y;
            }
          }
        }
      }
    }
#pragma unroll
    for (int j = 0; j < COUT; ++j) {
#pragma unroll
      for (int s = 16; s > 0; s >>= 1) acc[j] += __shfl_xor_sync(0xffffffffu, acc[j], s);
    }
    if (lane == 0) {
#pragma unroll
      for (int j = 0; j < COUT; ++j) y[pix * COUT + j] = __float2half_rn(acc[j] + (bias ? __half2float(bias[j]) : 0.f));
    }
  }
}

// ---- nearest-neighbour 2x up-sampling ---------------------------------------------
__global__ void upsample2x_kernel(const uint4* __restrict__ x, uint4* __restrict__ y, int B, int H, int W, int vecs) {
  pdl_launch_dependents();
  pdl_wait();
  const long long total = (long long)B * (2 * H) * (2 * W) * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const int v = i % vecs;
    const long long pix = i / vecs;
    const int ox = pix % (2 * W);
    const int oy = (pix / (2 * W)) % (2 * H);
    const int img = pix / (4ll * W * H);
    y[i] = x[(((long long)img * H + (oy >> 1)) * W + (ox >> 1)) * vecs + v];
  }
}

// ---- LayerNorm over the last axis, one warp per row --------------------------------
__global__ void layernorm_kernel(const __half* __restrict__ x, __half* __restrict__ y, const __half* __restrict__ gamma,
                                 const __half* __restrict__ beta, long long rows, int C, float eps, int w_static) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31;
  const int wpb = blockDim.x / 32;
  const int vecs = C / 8;
  // scale and shift of this lane's columns; when they are model weights they are fetched while
  // the previous kernel is still running
  uint4 gu[6], bu[6];
  auto load_affine = [&]() {
#pragma unroll
    for (int it = 0; it < 6; ++it) {
      const int v = lane + 32 * it;
      if (v < vecs) {
        gu[it] = *reinterpret_cast<const uint4*>(gamma + v * 8);
        bu[it] = *reinterpret_cast<const uint4*>(beta + v * 8);
      }
    }
  };
  if (w_static) load_affine();
  pdl_wait();
  if (!w_static) load_affine();
  for (long long r = blockIdx.x * (long long)wpb + (threadIdx.x >> 5); r < rows; r += (long long)gridDim.x * wpb) {
    const __half* xr = x + r * C;
    float vals[8 * 6];  // up to C = 1536: six 16-byte vectors per lane
    float s = 0.f;
#pragma unroll
    for (int it = 0; it < 6; ++it) {
      const int v = lane + 32 * it;
      if (v < vecs) {
        const uint4 u = *reinterpret_cast<const uint4*>(xr + v * 8);
        const __half2* h = reinterpret_cast<const __half2*>(&u);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 f = __half22float2(h[j]);
          vals[it * 8 + 2 * j] = f.x, vals[it * 8 + 2 * j + 1] = f.y;
          s += f.x + f.y;
        }
      } else {
#pragma unroll
        for (int j = 0; j < 8; ++j) vals[it * 8 + j] = 0.f;
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    const float mean = s / C;
    float q = 0.f;
#pragma unroll
    for (int it = 0; it < 6; ++it) {
      if (lane + 32 * it < vecs) {
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          const float d = vals[it * 8 + j] - mean;
          q += d * d;
        }
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) q += __shfl_xor_sync(0xffffffffu, q, o);
    const float rstd = rsqrtf(q / C + eps);
#pragma unroll
    for (int it = 0; it < 6; ++it) {
      const int v = lane + 32 * it;
      if (v < vecs) {
        const __half2* gh = reinterpret_cast<const __half2*>(&gu[it]);
        const __half2* bh = reinterpret_cast<const __half2*>(&bu[it]);
        uint4 o;
        __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          const float2 g = __half22float2(gh[j]), b = __half22float2(bh[j]);
          oh[j] = __floats2half2_rn((vals[it * 8 + 2 * j] - mean) * rstd * g.x + b.x,
                                    (vals[it * 8 + 2 * j + 1] - mean) * rstd * g.y + b.y);
        }
        *reinterpret_cast<uint4*>(y + r * C + v * 8) = o;
      }
    }
  }
}

// ---- GEGLU: out[m, f] = h[m, f] * gelu(h[m, F + f]) ----------------------------------
__global__ void geglu_kernel(const __half* __restrict__ h, __half* __restrict__ out, long long rows, int F) {
  pdl_launch_dependents();
  pdl_wait();
  const int vecs = F / 8;
  const long long total = rows * vecs;
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
    const long long r = i / vecs;
    const int v = i % vecs;
    const uint4 a = *reinterpret_cast<const uint4*>(h + r * 2 * F + v * 8);
    const uint4 g = *reinterpret_cast<const uint4*>(h + r * 2 * F + F + v * 8);
    const __half2* ah = reinterpret_cast<const __half2*>(&a);
    const __half2* gh = reinterpret_cast<const __half2*>(&g);
    uint4 o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const float2 x = __half22float2(ah[j]), t = __half22float2(gh[j]);
      const float g0 = 0.5f * t.x * (1.f + erff(t.x * 0.70710678118654752f));
      const float g1 = 0.5f * t.y * (1.f + erff(t.y * 0.70710678118654752f));
      oh[j] = __floats2half2_rn(x.x * g0, x.y * g1);
    }
    *reinterpret_cast<uint4*>(out + r * F + v * 8) = o;
  }
}

// ---- guidance combine + Euler update + input scaling for the next step -------------------
// eps [2][n] fp16 (row 0 unconditional, row 1 conditional); latents [n] fp32 updated in place;
// next_input [2][n] fp16 = latents / sqrt(sigma_next^2 + 1), the same in both rows.
__global__ void cfg_euler_kernel(const __half* __restrict__ eps, float* __restrict__ latents, __half* __restrict__ next_input,
                                 long long n, float guidance, float dsigma, float in_scale) {
  pdl_launch_dependents();
  pdl_wait();
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
    const float e0 = __half2float(eps[i]), e1 = __half2float(eps[n + i]);
    const float e = e0 + guidance * (e1 - e0);
    const float x = latents[i] + e * dsigma;
    latents[i] = x;
    const __half h = __float2half_rn(x * in_scale);
    next_input[i] = h;
    next_input[n + i] = h;
  }
}

static int grid_for(long long work_items, int threads) {
  long long blocks = (work_items + threads - 1) / threads;
  const long long cap = (long long)sm_count() * 16;
  if (blocks > cap) blocks = cap;
  if (blocks < 1) blocks = 1;
  return (int)blocks;
}
static bool al16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace bxl

using namespace bxl;

extern "C" int bxl_halo_pack_f16(const void* x, long long img_stride, void* out, int B, int H, int W, int C, int pad,
                                 void* stream) {
  if (!x || !out) return fail(kErrInvalidArg, "bxl_halo_pack_f16: null pointer");
  if (B <= 0 || H <= 0 || W <= 0 || C <= 0 || pad <= 0 || pad > H) return fail(kErrInvalidArg, "bxl_halo_pack_f16: bad extent");
  if (C % 8 || img_stride % 8 || !al16(x) || !al16(out)) return fail(kErrInvalidArg, "bxl_halo_pack_f16: C, stride and pointers must be 16-byte granular");
  const long long row_v = (long long)W * C / 8;
  const long long total = 2ll * B * pad * row_v;
  return launch_kernel("halo_pack_kernel launch", halo_pack_kernel, dim3(grid_for(total, 256)), dim3(256), 0, (cudaStream_t)stream, 1,
                       static_cast<const uint4*>(x), img_stride / 8, static_cast<uint4*>(out), B, H, row_v, pad);
}

extern "C" int bxl_conv3x3_direct_f16(const void* x, long long x_img_stride, const void* top, const void* bot,
                                      long long halo_img_stride, const void* w_packed, const void* bias, void* y, int B,
                                      int C_in, int C_out, int H, int W, void* stream) {
  if (!x || !w_packed || !y) return fail(kErrInvalidArg, "bxl_conv3x3_direct_f16: null pointer");
  if (B <= 0 || H <= 0 || W <= 0 || C_in <= 0 || C_out <= 0) return fail(kErrInvalidArg, "bxl_conv3x3_direct_f16: bad extent");
  cudaStream_t s = (cudaStream_t)stream;
  if (C_in <= 16 && C_out % 8 == 0) {
    const size_t smem = (size_t)C_out * 9 * C_in * sizeof(float);
    if (smem > 200 * 1024) return fail(kErrTooLarge, "bxl_conv3x3_direct_f16: weights do not fit shared memory");
    static bool configured[64] = {};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
      if (int rc = check_cuda(cudaFuncSetAttribute(conv3x3_small_cin_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024),
                              "cudaFuncSetAttribute(conv_small_cin)"))
        return rc;
      configured[dev] = true;
    }
    // C_in == 4 with 8-byte aligned rows: four pixels per thread
    if (C_in == 4 && al16(w_packed) && x_img_stride % 4 == 0 && halo_img_stride % 4 == 0 && (reinterpret_cast<uintptr_t>(x) & 7u) == 0 &&
        (!top || (reinterpret_cast<uintptr_t>(top) & 7u) == 0) && (!bot || (reinterpret_cast<uintptr_t>(bot) & 7u) == 0) && al16(y)) {
      static bool configured4[64] = {};
      if (dev >= 0 && dev < 64 && !configured4[dev]) {
        if (int rc = check_cuda(cudaFuncSetAttribute(conv3x3_cin4_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024),
                                "cudaFuncSetAttribute(conv_cin4)"))
          return rc;
        configured4[dev] = true;
      }
      const long long total4 = (long long)B * H * ((W + 3) / 4) * (C_out / 8);
      int blocks4 = grid_for(total4, 256);
      if (blocks4 > sm_count() * 4) blocks4 = sm_count() * 4;  // weights are staged once per CTA
      conv3x3_cin4_kernel<<<blocks4, 256, smem, s>>>(static_cast<const __half*>(x), x_img_stride, static_cast<const __half*>(top),
                                                     static_cast<const __half*>(bot), halo_img_stride,
                                                     static_cast<const __half*>(w_packed), static_cast<const __half*>(bias),
                                                     static_cast<__half*>(y), B, C_out, H, W);
      return check_cuda(cudaGetLastError(), "conv3x3_cin4 launch");
    }
    const long long total = (long long)B * H * W * (C_out / 8);
    int blocks = grid_for(total, 256);
    if (blocks > sm_count() * 4) blocks = sm_count() * 4;  // weights are staged once per CTA
    conv3x3_small_cin_kernel<<<blocks, 256, smem, s>>>(static_cast<const __half*>(x), x_img_stride,
                                                       static_cast<const __half*>(top), static_cast<const __half*>(bot),
                                                       halo_img_stride, static_cast<const __half*>(w_packed),
                                                       static_cast<const __half*>(bias), static_cast<__half*>(y), B, C_in,
                                                       C_out, H, W);
  } else if (C_out == 4 && C_in % 8 == 0) {
    if (!al16(x) || (top && !al16(top)) || (bot && !al16(bot)) || !al16(w_packed) || x_img_stride % 8 || halo_img_stride % 8)
      return fail(kErrInvalidArg, "bxl_conv3x3_direct_f16: pointers must be 16-byte aligned");
    const long long total = (long long)B * H * W;
    conv3x3_small_cout_kernel<4><<<grid_for(total * 32, 256), 256, 0, s>>>(
        static_cast<const __half*>(x), x_img_stride, static_cast<const __half*>(top), static_cast<const __half*>(bot),
        halo_img_stride, static_cast<const __half*>(w_packed), static_cast<const __half*>(bias), static_cast<__half*>(y), B,
        C_in, H, W);
  } else {
    return fail(kErrUnsupported, "bxl_conv3x3_direct_f16: C_in=%d C_out=%d not covered (C_in<=16 or C_out==4)", C_in, C_out);
  }
  return check_cuda(cudaGetLastError(), "conv3x3_direct launch");
}

extern "C" int bxl_upsample2x_f16(const void* x, void* y, int B, int H, int W, int C, void* stream) {
  if (!x || !y || B <= 0 || H <= 0 || W <= 0 || C <= 0 || C % 8 || !al16(x) || !al16(y))
    return fail(kErrInvalidArg, "bxl_upsample2x_f16: bad argument");
  const long long total = (long long)B * 4 * H * W * (C / 8);
  return launch_kernel("upsample2x_kernel launch", upsample2x_kernel, dim3(grid_for(total, 256)), dim3(256), 0, (cudaStream_t)stream, 1,
                       static_cast<const uint4*>(x), static_cast<uint4*>(y), B, H, W, C / 8);
}

extern "C" int bxl_layernorm_f16(const void* x, void* y, const void* gamma, const void* beta, long long rows, int C, float eps,
                                 void* stream) {
  if (!x || !y || !gamma || !beta || rows <= 0 || C <= 0) return fail(kErrInvalidArg, "bxl_layernorm_f16: bad argument");
  if (C % 8 || C > 1536 || !al16(x) || !al16(y) || !al16(gamma) || !al16(beta))
    return fail(kErrUnsupported, "bxl_layernorm_f16: C=%d must be a multiple of 8, at most 1536, pointers 16-byte aligned", C);
  return launch_kernel("layernorm_kernel launch", layernorm_kernel, dim3(grid_for(rows * 32, 256)), dim3(256), 0, (cudaStream_t)stream, 1,
                       static_cast<const __half*>(x), static_cast<__half*>(y), static_cast<const __half*>(gamma),
                       static_cast<const __half*>(beta), rows, C, eps, static_weights() ? 1 : 0);
}

extern "C" int bxl_geglu_f16(const void* h, void* out, long long rows, int F, void* stream) {
  if (!h || !out || rows <= 0 || F <= 0 || F % 8 || !al16(h) || !al16(out)) return fail(kErrInvalidArg, "bxl_geglu_f16: bad argument");
  return launch_kernel("geglu_kernel launch", geglu_kernel, dim3(grid_for(rows * (F / 8), 256)), dim3(256), 0, (cudaStream_t)stream, 1,
                       static_cast<const __half*>(h), static_cast<__half*>(out), rows, F);
}

extern "C" int bxl_cfg_euler_step(const void* eps, float* latents, void* next_input, long long n, float guidance, float sigma,
                                  float sigma_next, void* stream) {
  if (!eps || !latents || !next_input || n <= 0) return fail(kErrInvalidArg, "bxl_cfg_euler_step: bad argument");
  const float in_scale = 1.f / sqrtf(sigma_next * sigma_next + 1.f);
  return launch_kernel("cfg_euler_kernel launch", cfg_euler_kernel, dim3(grid_for(n, 256)), dim3(256), 0, (cudaStream_t)stream, 1,
                       static_cast<const __half*>(eps), latents, static_cast<__half*>(next_input), n, guidance,
                       sigma_next - sigma, in_scale);
}
