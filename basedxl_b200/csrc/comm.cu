// Strip-to-strip exchange over peer memory (NVLink / NVSwitch), for the points of a denoising step
// where every strip needs the others' FRESH data before it can go on: the per-layer exchanges of
// the synchronous steps (halo rows, GroupNorm moments, K/V) and the assembly of the step's output
// from the strips.
//
// One launch does what a blocking all-gather does: every rank copies its contribution from its own
// memory into the place reserved for it in each peer's memory (plain stores through the peer
// mapping; no tensor-map copies, no multicast), then the ranks meet at a flag barrier: the last CTA
// of the grid publishes the exchange's sequence number in each peer's flag word for this rank
// (release, system scope) and waits until every peer's word in its own flag array has reached the
// same number (acquire, system scope).  When the kernel ends, every peer's contribution is in this
// rank's memory and visible to the kernels that follow on the stream.
//
// Every rank of a group must launch the same sequence of exchanges on one stream per group.  A
// peer may run at most one exchange ahead, so two CONSECUTIVE exchanges of a group must not target
// the same destination range unless the second one is launched with `handshake`: it then first
// waits until every peer has reached the same exchange (i.e. has finished the kernels that read
// the previous contents) before it overwrites anything.
//
// The wait is bounded: after `wait_ns` the kernel records {wait timeout, site 900 + peer} in the
// device status word and returns; bxl_device_status() reports it.  Roofline: NVLink; algorithmic
// bytes = (peers - 1) x contribution per rank.
#include "bxl_common.cuh"
#include "bxl_host.h"
#include "../../include/basedxl_b200.h"

namespace bxl {

constexpr int kCommMaxPeers = 8;
// layout of a group's control words (uint32, in memory every peer can write):
//   [0, 8)   "data sent" sequence numbers, word p written by peer p
//   [8, 16)  "ready to receive" sequence numbers (handshake), word p written by peer p
//   [16]     this rank's sequence number of the last exchange   [17] CTA ticket (both local use only)
constexpr int kCtlSent = 0, kCtlReady = 8, kCtlSeq = 16, kCtlTicket = 17;

struct ExchangeParams {
  const uint4* src;               // this rank's contribution (local memory)
  uint4* dst[kCommMaxPeers];      // its place in peer p's memory; null = nothing to copy for p
  long long n_vec;                // 16-byte vectors
  int n_peers, own;
  unsigned* ctl;                  // this rank's control words
  unsigned* ctl_peer[kCommMaxPeers];  // peer p's control words (peer memory)
  int handshake;
  unsigned long long wait_ns;
  int* dev_status;
};

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// Bounded wait until *word has reached `seq` (sequence numbers wrap: compare as a signed difference).
__device__ __forceinline__ bool wait_seq(const unsigned* word, unsigned seq, unsigned long long limit_ns, int* dev_status, int site) {
  if (static_cast<int>(ld_acquire_sys(word) - seq) >= 0) return true;
  const unsigned long long t0 = global_timer_ns();
  unsigned spins = 0;
  while (true) {
    if (static_cast<int>(ld_acquire_sys(word) - seq) >= 0) return true;
    if ((++spins & 63u) == 0u && global_timer_ns() - t0 > limit_ns) {
      if (atomicCAS(&dev_status[0], kDevOk, kDevWaitTimeout) == kDevOk) {
        dev_status[1] = site;
        dev_status[2] = static_cast<int>(blockIdx.x);
      }
      __threadfence();
      return false;
    }
  }
}

__global__ void __launch_bounds__(256) exchange_kernel(const ExchangeParams p) {
  pdl_launch_dependents();
  pdl_wait();
  __shared__ int s_ok;
  if (p.handshake) {
    // nobody may overwrite a range its owner still reads: every rank announces that it has
    // reached this exchange (its earlier kernels are done), and waits for all the others
    if (threadIdx.x == 0) {
      const unsigned seq = p.ctl[kCtlSeq] + 1u;
      int ok = 1;
      if (blockIdx.x == 0) {
        __threadfence_system();
        for (int q = 0; q < p.n_peers; ++q)
          if (q != p.own) st_release_sys(p.ctl_peer[q] + kCtlReady + p.own, seq);
      }
      for (int q = 0; q < p.n_peers && ok; ++q)
        if (q != p.own) ok = wait_seq(p.ctl + kCtlReady + q, seq, p.wait_ns, p.dev_status, 800 + q) ? 1 : 0;
      s_ok = ok;
    }
    __syncthreads();
    if (!s_ok) return;  // timed out: touch nothing of the peers'
  }
  // ---- contribution -> every peer
  for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < p.n_vec; i += (long long)gridDim.x * blockDim.x) {
    const uint4 v = p.src[i];
#pragma unroll
    for (int q = 0; q < kCommMaxPeers; ++q)
      if (q < p.n_peers && p.dst[q]) p.dst[q][i] = v;
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x != 0) return;
  // ---- the last CTA to get here signals the peers and waits for theirs
  const unsigned t = atomicAdd(p.ctl + kCtlTicket, 1u);
  if (t != gridDim.x - 1) return;
  p.ctl[kCtlTicket] = 0;
  const unsigned seq = p.ctl[kCtlSeq] + 1u;
  p.ctl[kCtlSeq] = seq;
  __threadfence_system();
  for (int q = 0; q < p.n_peers; ++q)
    if (q != p.own) st_release_sys(p.ctl_peer[q] + kCtlSent + p.own, seq);
  for (int q = 0; q < p.n_peers; ++q)
    if (q != p.own && !wait_seq(p.ctl + kCtlSent + q, seq, p.wait_ns, p.dev_status, 900 + q)) return;
}

}  // namespace bxl

using namespace bxl;

extern "C" long long bxl_comm_ctl_bytes(void) { return 32 * sizeof(unsigned); }

// ---- mapping a peer process's buffer (CUDA IPC) --------------------------------------
typedef CUresult (*GetAddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);

extern "C" int bxl_comm_ipc_export(const void* ptr, unsigned char* handle64, long long* offset_bytes) {
  if (!ptr || !handle64 || !offset_bytes) return fail(kErrInvalidArg, "bxl_comm_ipc_export: null argument");
  static GetAddressRangeFn get_range = nullptr;
  if (!get_range) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    const cudaError_t e = cudaGetDriverEntryPoint("cuMemGetAddressRange", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess || q != cudaDriverEntryPointSuccess || !fn)
      return fail(kErrCuda, "bxl_comm_ipc_export: cuMemGetAddressRange entry point unavailable (%s)", cudaGetErrorString(e));
    get_range = reinterpret_cast<GetAddressRangeFn>(fn);
  }
  CUdeviceptr base = 0;
  size_t size = 0;
  const CUresult r = get_range(&base, &size, reinterpret_cast<CUdeviceptr>(ptr));
  if (r != CUDA_SUCCESS) return fail(kErrCuda, "bxl_comm_ipc_export: cuMemGetAddressRange failed with CUresult %d", (int)r);
  cudaIpcMemHandle_t h;
  static_assert(sizeof(h) == 64, "IPC handles are 64 bytes");
  if (int rc = check_cuda(cudaIpcGetMemHandle(&h, reinterpret_cast<void*>(base)), "cudaIpcGetMemHandle")) return rc;
  memcpy(handle64, &h, 64);
  *offset_bytes = static_cast<long long>(reinterpret_cast<CUdeviceptr>(ptr) - base);
  return kOk;
}

extern "C" int bxl_comm_ipc_open(const unsigned char* handle64, void** base_out) {
  if (!handle64 || !base_out) return fail(kErrInvalidArg, "bxl_comm_ipc_open: null argument");
  cudaIpcMemHandle_t h;
  memcpy(&h, handle64, 64);
  void* p = nullptr;
  // opened with the CURRENT device as the one that will access the memory: peer access between it
  // and the owning device is switched on as part of the mapping
  if (int rc = check_cuda(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle")) return rc;
  *base_out = p;
  return kOk;
}

extern "C" int bxl_comm_ipc_close(void* base) {
  if (!base) return kOk;
  return check_cuda(cudaIpcCloseMemHandle(base), "cudaIpcCloseMemHandle");
}

extern "C" int bxl_comm_exchange(const void* src, void* const* peer_dst, long long nbytes, void* ctl, void* const* peer_ctl,
                                 int n_peers, int own, int handshake, double wait_seconds, void* stream) {
  if (n_peers < 1 || n_peers > kCommMaxPeers || own < 0 || own >= n_peers)
    return fail(kErrInvalidArg, "bxl_comm_exchange: %d peers / own %d (1..%d peers)", n_peers, own, kCommMaxPeers);
  if (!ctl || !peer_ctl || !peer_dst) return fail(kErrInvalidArg, "bxl_comm_exchange: null table");
  if (nbytes < 0 || nbytes % 16) return fail(kErrInvalidArg, "bxl_comm_exchange: nbytes=%lld must be a non-negative multiple of 16", nbytes);
  if (nbytes > 0 && (!src || (reinterpret_cast<uintptr_t>(src) & 15u))) return fail(kErrInvalidArg, "bxl_comm_exchange: src must be 16-byte aligned");
  if (!(wait_seconds > 0.0) || wait_seconds > 60.0) return fail(kErrInvalidArg, "bxl_comm_exchange: wait_seconds must lie in (0, 60]");
  int* st = device_status_ptr();
  if (!st) return fail(kErrCuda, "bxl_comm_exchange: no device status word");
  ExchangeParams p;
  memset(&p, 0, sizeof(p));
  p.src = static_cast<const uint4*>(src);
  p.n_vec = nbytes / 16;
  p.n_peers = n_peers, p.own = own;
  p.ctl = static_cast<unsigned*>(ctl);
  for (int q = 0; q < n_peers; ++q) {
    if (peer_dst[q] && (reinterpret_cast<uintptr_t>(peer_dst[q]) & 15u))
      return fail(kErrInvalidArg, "bxl_comm_exchange: destination %d is not 16-byte aligned", q);
    p.dst[q] = static_cast<uint4*>(peer_dst[q]);
    if (q != own && !peer_ctl[q]) return fail(kErrInvalidArg, "bxl_comm_exchange: control words of peer %d missing", q);
    p.ctl_peer[q] = static_cast<unsigned*>(peer_ctl[q]);
  }
  p.handshake = handshake ? 1 : 0;
  p.wait_ns = static_cast<unsigned long long>(wait_seconds * 1e9);
  p.dev_status = st;
  // enough CTAs to keep several NVLink stores in flight per peer, few enough to leave the SMs to
  // the compute kernels around it
  long long blocks = (p.n_vec + 256 * 8 - 1) / (256 * 8);
  if (blocks > 32) blocks = 32;
  if (blocks < 1) blocks = 1;
  return launch_kernel("exchange_kernel launch", exchange_kernel, dim3((unsigned)blocks), dim3(256), 0, (cudaStream_t)stream, 1, p);
}
