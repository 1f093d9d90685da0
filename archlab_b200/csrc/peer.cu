// Fused collective + optimizer kernels over NVLink peer memory (ZeRO-1 data parallelism).
//
// Every rank keeps its gradient buffers and bf16 shadow weights in symmetric memory (same offset
// on every GPU, mapped into every process), so a kernel can load a peer's gradients and store into
// a peer's shadows directly.  One launch per tensor then does what the reference's distributed
// optimizer does with three NCCL phases (src/archlab/optimizers/speedrun.py:520-755):
//
//   reduce-scatter   : the owner of a slice LOADS that slice from all `world` gradient buffers
//   cast/scale/update: mean, AdamW (or Muon momentum) in registers
//   all-gather       : the owner STORES the new bf16 weights into every rank's shadow buffer
//
// so each gradient byte crosses NVLink once and no intermediate buffer is written.  Ordering
// between ranks comes from `peer_barrier_kernel` (flags in symmetric memory, release/acquire at
// system scope, bounded wait that reports through the status word instead of hanging).
#include "ptx.cuh"
#include "host_util.h"
#include "peer.h"

namespace nga {

constexpr int kMaxWorld = 16;

struct PeerPtrs {
  void* p[kMaxWorld];
};

__device__ __forceinline__ void st_release_sys(int* addr, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(addr), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* addr) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(addr) : "memory");
  return v;
}

// Each rank writes `epoch` into slot [rank] of every peer's flag array, then waits until all slots
// of its own array have reached `epoch`.  One block, `world` active threads.
__global__ void peer_barrier_kernel(PeerPtrs flags, int rank, int world, int epoch, int* status,
                                    unsigned long long budget_ns) {
  const int t = threadIdx.x;
  __threadfence_system();
  if (t < world) {
    st_release_sys(reinterpret_cast<int*>(flags.p[t]) + rank, epoch);
    const int* mine = reinterpret_cast<const int*>(flags.p[rank]) + t;
    const unsigned long long t0 = globaltimer_ns();
    unsigned it = 0;
    // once a wait of this process has expired the step is lost anyway: later barriers do not wait again, so the host
    // reaches its next status check after one budget instead of one budget per barrier
    const bool lost = *reinterpret_cast<volatile int*>(status) != 0;
    while (!lost && ld_acquire_sys(mine) < epoch) {
      if ((++it & 255u) == 0u && globaltimer_ns() - t0 > budget_ns) {
        atomicCAS(status, 0, kErrPeerTimeout);
        break;
      }
    }
  }
  __threadfence_system();
}

// ------------------------------------------------------------------------------------------------
// Fused reduce-scatter + AdamW + all-gather over an owned element range [e0, e0 + n).
//   grads[r]   : fp32 gradient buffer of rank r (full tensor, symmetric)
//   shadows[r] : bf16 shadow buffer of rank r (full tensor, symmetric)
//   p, m, v    : this rank's fp32 master / moments for the OWNED slice only (n elements)
// ------------------------------------------------------------------------------------------------
__global__ void peer_adamw_kernel(PeerPtrs grads, PeerPtrs shadows, float* __restrict__ p,
                                  float* __restrict__ m, float* __restrict__ v, long long e0, long long n,
                                  int world, float lr, float beta1, float beta2, float eps, float wd,
                                  float inv_bias1, float inv_bias2, int cautious) {
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= n) return;
  float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
  for (int r = 0; r < world; ++r) {
    const float4 x = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + e0 + i);
    g.x += x.x; g.y += x.y; g.z += x.z; g.w += x.w;
  }
  const float inv = 1.f / world;
  float gp[4] = {g.x * inv, g.y * inv, g.z * inv, g.w * inv};
  float4 pv = *reinterpret_cast<float4*>(p + i);
  float4 mv = *reinterpret_cast<float4*>(m + i);
  float4 vv = *reinterpret_cast<float4*>(v + i);
  float* pp = reinterpret_cast<float*>(&pv);
  float* mp = reinterpret_cast<float*>(&mv);
  float* vp = reinterpret_cast<float*>(&vv);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    mp[k] += (1.f - beta1) * (gp[k] - mp[k]);
    vp[k] += (1.f - beta2) * (gp[k] * gp[k] - vp[k]);
    const float upd = mp[k] / (sqrtf(vp[k] * inv_bias2) + eps);
    if (cautious) {
      if (upd * pp[k] >= 0.f) pp[k] -= lr * wd * pp[k];
    } else {
      pp[k] *= 1.f - lr * wd;
    }
    pp[k] -= lr * inv_bias1 * upd;
  }
  *reinterpret_cast<float4*>(p + i) = pv;
  *reinterpret_cast<float4*>(m + i) = mv;
  *reinterpret_cast<float4*>(v + i) = vv;
  uint2 u;
  u.x = pack_bf16(pp[0], pp[1]);
  u.y = pack_bf16(pp[2], pp[3]);
  for (int r = 0; r < world; ++r)
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(shadows.p[r]) + e0 + i) = u;
}

// Fused reduce-scatter + Muon Nesterov momentum for the owned matrices of a stacked group.
//   g_out (fp32, local, K_own * per) receives the Nesterov gradient; norm2[k] its squared norm.
__global__ void peer_muon_momentum_kernel(PeerPtrs grads, float* __restrict__ g_out, float* __restrict__ m,
                                          float* __restrict__ norm2, long long e0, long long per, int world,
                                          float mu) {
  __shared__ float red[8];
  const long long base = (long long)blockIdx.y * per;
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  float acc = 0.f;
  if (i < per) {
    float4 g = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
    for (int r = 0; r < world; ++r) {
      const float4 x = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(grads.p[r]) + e0 + base + i);
      g.x += x.x; g.y += x.y; g.z += x.z; g.w += x.w;
    }
    const float inv = 1.f / world;
    float gp[4] = {g.x * inv, g.y * inv, g.z * inv, g.w * inv};
    float4 mv = *reinterpret_cast<float4*>(m + base + i);
    float* mp = reinterpret_cast<float*>(&mv);
#pragma unroll
    for (int k = 0; k < 4; ++k) {
      mp[k] += (1.f - mu) * (gp[k] - mp[k]);
      gp[k] += mu * (mp[k] - gp[k]);
      acc += gp[k] * gp[k];
    }
    *reinterpret_cast<float4*>(g_out + base + i) = make_float4(gp[0], gp[1], gp[2], gp[3]);
    *reinterpret_cast<float4*>(m + base + i) = mv;
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = acc;
  __syncthreads();
  if (threadIdx.x == 0) {
    float t = 0.f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) t += red[w];
    atomicAdd(norm2 + blockIdx.y, t);
  }
}

// Muon final step for the owned matrices with the all-gather fused in: the new bf16 weights are
// stored into every rank's shadow buffer at element offset e0.
__global__ void peer_muon_apply_kernel(float* __restrict__ p, const __nv_bfloat16* __restrict__ x,
                                       const float* __restrict__ scale, PeerPtrs shadows, long long e0, int m,
                                       int n, int per_row, int world, float lr, float wd) {
  const long long per = (long long)m * n;
  const long long base = (long long)blockIdx.y * per;
  const long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (i >= per) return;
  const int r0 = int(i / n), c = int(i % n);
  float4 pv = *reinterpret_cast<float4*>(p + base + i);
  const uint2 xv = *reinterpret_cast<const uint2*>(x + base + i);
  const float2 x01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv.x));
  const float2 x23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&xv.y));
  const float xs[4] = {x01.x, x01.y, x23.x, x23.y};
  float* pp = reinterpret_cast<float*>(&pv);
#pragma unroll
  for (int k = 0; k < 4; ++k) {
    const float sc = per_row ? scale[(long long)blockIdx.y * m + r0] : scale[(long long)blockIdx.y * n + c + k];
    const float u = __bfloat162float(__float2bfloat16(xs[k] * sc));
    const float decay = (u * pp[k] >= 0.f) ? lr * wd * pp[k] : 0.f;
    pp[k] -= lr * u + decay;
  }
  *reinterpret_cast<float4*>(p + base + i) = pv;
  uint2 u2;
  u2.x = pack_bf16(pp[0], pp[1]);
  u2.y = pack_bf16(pp[2], pp[3]);
  for (int r = 0; r < world; ++r)
    *reinterpret_cast<uint2*>(reinterpret_cast<__nv_bfloat16*>(shadows.p[r]) + e0 + base + i) = u2;
}

static PeerPtrs make_ptrs(const long long* host_ptrs, int world) {
  PeerPtrs pp;
  for (int i = 0; i < kMaxWorld; ++i) pp.p[i] = i < world ? reinterpret_cast<void*>(host_ptrs[i]) : nullptr;
  return pp;
}

}  // namespace nga

using namespace nga;
#define ST(s) reinterpret_cast<cudaStream_t>(s)

// How long a kernel waits for a flag another GPU writes before it gives up and reports kErrPeerTimeout through the
// status word (default 2 s).  A launch parameter, so a health check or a test can ask for a short wait.
static unsigned long long g_peer_wait_budget_ns = kWaitBudgetNs;
extern "C" void nga_set_peer_wait_budget_ns(unsigned long long ns) { g_peer_wait_budget_ns = ns ? ns : kWaitBudgetNs; }
extern "C" unsigned long long nga_peer_wait_budget_ns(void) { return g_peer_wait_budget_ns; }

extern "C" int nga_peer_barrier(const long long* flag_ptrs, int rank, int world, int epoch, int* status,
                                void* stream) {
  if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return -1;
  peer_barrier_kernel<<<1, 32, 0, ST(stream)>>>(make_ptrs(flag_ptrs, world), rank, world, epoch, status,
                                                g_peer_wait_budget_ns);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_peer_adamw(const long long* grad_ptrs, const long long* shadow_ptrs, float* p, float* m,
                              float* v, long long e0, long long n, int world, float lr, float beta1, float beta2,
                              float eps, float wd, int step, int cautious, void* stream) {
  if (world < 1 || world > kMaxWorld || n <= 0 || (n % 4) || (e0 % 4) || step < 1) return -1;
  const float inv_b1 = 1.f / (1.f - powf(beta1, (float)step));
  const float inv_b2 = 1.f / (1.f - powf(beta2, (float)step));
  peer_adamw_kernel<<<(unsigned)((n / 4 + 255) / 256), 256, 0, ST(stream)>>>(
      make_ptrs(grad_ptrs, world), make_ptrs(shadow_ptrs, world), p, m, v, e0, n, world, lr, beta1, beta2, eps,
      wd, inv_b1, inv_b2, cautious);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_peer_muon_momentum(const long long* grad_ptrs, float* g_out, float* m, float* norm2,
                                      long long e0, int K, long long per, int world, float mu, void* stream) {
  if (world < 1 || world > kMaxWorld || K <= 0 || per <= 0 || (per % 4) || (e0 % 4)) return -1;
  cudaMemsetAsync(norm2, 0, sizeof(float) * K, ST(stream));
  dim3 grid((unsigned)((per / 4 + 255) / 256), K);
  peer_muon_momentum_kernel<<<grid, 256, 0, ST(stream)>>>(make_ptrs(grad_ptrs, world), g_out, m, norm2, e0, per,
                                                          world, mu);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}

extern "C" int nga_peer_muon_apply(float* p, const void* x, const float* scale, const long long* shadow_ptrs,
                                   long long e0, int K, int m, int n, int per_row, int world, float lr, float wd,
                                   void* stream) {
  if (world < 1 || world > kMaxWorld || K <= 0 || m <= 0 || n <= 0 || (n % 4) || (e0 % 4)) return -1;
  const long long per = (long long)m * n;
  dim3 grid((unsigned)((per / 4 + 255) / 256), K);
  peer_muon_apply_kernel<<<grid, 256, 0, ST(stream)>>>(p, reinterpret_cast<const __nv_bfloat16*>(x), scale,
                                                       make_ptrs(shadow_ptrs, world), e0, m, n, per_row, world, lr,
                                                       wd);
  count_launch();
  NGA_CHECK_LAUNCH();
  return 0;
}
