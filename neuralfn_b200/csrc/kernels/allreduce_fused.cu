// One-shot all-reduce of a small [rows, N] bf16 activation across the GPUs of one NVSwitch
// domain, fused with what follows a row-parallel projection in a decode step: residual add
// and (optionally) the next RMS norm. Latency is what matters at these sizes (32 x 6656
// bf16 = 416 KB), so there is exactly one signal exchange and one pass over the data:
//
//   1. the partial result of this rank already sits in a symmetric buffer (the projection
//      kernel wrote it there); CTA 0 raises this rank's flag in every peer's control block;
//   2. every CTA waits (bounded) until all peers have raised theirs;
//   3. each CTA owns whole rows: it sums the `world` partials - either with plain 16-byte
//      loads from each peer's buffer over NVLink, or with one multimem.ld_reduce per 16 bytes
//      on the multicast address of the buffer so the switch does the addition - adds the
//      residual, stores the new residual stream, and normalises the row for the next layer;
//   4. CTA 0's peers must not overwrite their partial buffer while others still read it: a
//      second flag round ("done reading") closes the call, checked by the NEXT call on the
//      same buffer before a rank's producer may overwrite it (callers alternate two buffers,
//      the check is nfn_allreduce_wait_readers).
//
// The reference has no counterpart (single GPU); its decode epilogues that this replaces are
// the gated / residual projection epilogues of glimmer_k_mmq.cu:2521-2637.
#include "common.h"
#include "nfn_kernels.h"
#include "sm100_ptx.cuh"

namespace nfn {

constexpr int AR_MAX_WORLD = 8, AR_MAX_THREADS = 1024;

struct ArParams {
  const __nv_bfloat16* peer[AR_MAX_WORLD];
  const __nv_bfloat16* mc;  // multicast address of the same buffer, or null
  int* ctrl;                // local control block: [0, 8) partial-ready flags, [8, 16) done-reading flags
  int* peer_ctrl[AR_MAX_WORLD];
  int rank, world, epoch;
  const int* epoch_dev;
  int rows, n, ld;
  const __nv_bfloat16* bias;
  __nv_bfloat16* resid;  // in/out, may be null
  int ld_resid;
  const __nv_bfloat16* norm_weight;  // null: no norm, `out` receives the reduced (+resid) rows
  float eps;
  int centered;  // norm weight applied as (1 + w)
  // sandwich blocks: the reduced branch output is normalised with `post_weight` BEFORE it joins the
  // residual stream (null: not used)
  const __nv_bfloat16* post_weight;
  float post_eps;
  __nv_bfloat16* out;
  int ld_out;
  int* status;
  unsigned long long* trace;  // optional [5]: globaltimer at start / signalled / peers arrived / rows done / end (CTA 0)
};

__device__ __forceinline__ void ar_st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
// one fence, then a relaxed store per peer: a release store per peer would pay the system-scope fence `world` times
// (measured: 1.5 us each)
__device__ __forceinline__ void ar_fence_release_sys() { asm volatile("fence.acq_rel.sys;" ::: "memory"); }
__device__ __forceinline__ void ar_st_relaxed_sys(int* p, int v) {
  asm volatile("st.relaxed.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ar_ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 ld_peer_16(const void* p) {
  uint4 v;
  asm volatile("ld.relaxed.sys.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ uint4 multimem_sum_bf16x8(const void* mc) {
  uint4 v;
  asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
               : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
               : "l"(mc)
               : "memory");
  return v;
}

__device__ bool ar_wait_all(const int* flags, int world, int want, int* status) {
  const unsigned long long t0 = global_timer_ns();
  for (int r = 0; r < world; ++r) {
#pragma unroll 1
    for (uint32_t it = 0;; ++it) {
      if (ar_ld_acquire_sys(flags + r) - want >= 0) break;
      if ((it & 7u) == 7u) {
        if (global_timer_ns() - t0 > 10ull * kWaitLimitNs) {
          if (status) atomicCAS(status, 0, NFN_ERR_WAIT_PEER);
          return false;
        }
        __nanosleep(32);
      }
    }
  }
  return true;
}

__global__ void __launch_bounds__(AR_MAX_THREADS)
allreduce_resid_norm_kernel(const ArParams p) {
  __shared__ float red[AR_MAX_THREADS / 32];
  __shared__ int sh_ok;
  extern __shared__ float rowbuf[];  // n floats
  const int epoch = p.epoch + (p.epoch_dev ? *p.epoch_dev : 0);
  const bool tracer = p.trace && blockIdx.x == 0 && threadIdx.x == 0;
  if (tracer) p.trace[0] = global_timer_ns();
  if (threadIdx.x == 0) {
    // the partial rows were written by an earlier kernel of this stream: they are complete in this GPU's memory, and the
    // release at system scope orders them before the flag for the peers that acquire it
    if (blockIdx.x == 0) {
      ar_fence_release_sys();
      for (int r = 0; r < p.world; ++r) ar_st_relaxed_sys(p.peer_ctrl[r] + p.rank, epoch);
    }
    if (tracer) p.trace[1] = global_timer_ns();
    sh_ok = ar_wait_all(p.ctrl, p.world, epoch, p.status) ? 1 : 0;
    if (tracer) p.trace[2] = global_timer_ns();
  }
  __syncthreads();
  if (!sh_ok) return;

  const int vecs = p.n / 8;
  auto block_total = [&](float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();   // the previous use of `red` is over
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    float tot = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) tot += red[w];
    return tot;
  };
  auto add_resid_store = [&](int row, int v, float (&s)[8]) {
    __nv_bfloat16* rp = p.resid + (long long)row * p.ld_resid + v * 8;
    const uint4 u = *reinterpret_cast<const uint4*>(rp);
    const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
    s[0] += a.x; s[1] += a.y; s[2] += b.x; s[3] += b.y; s[4] += c.x; s[5] += c.y; s[6] += d.x; s[7] += d.y;
    uint4 o;
    o.x = pack_bf16x2(s[0], s[1]); o.y = pack_bf16x2(s[2], s[3]); o.z = pack_bf16x2(s[4], s[5]); o.w = pack_bf16x2(s[6], s[7]);
    *reinterpret_cast<uint4*>(rp) = o;
    // the norm sees the residual stream as stored (bf16)
    const float2 a2 = unpack_bf16x2(o.x), b2 = unpack_bf16x2(o.y), c2 = unpack_bf16x2(o.z), d2 = unpack_bf16x2(o.w);
    s[0] = a2.x; s[1] = a2.y; s[2] = b2.x; s[3] = b2.y; s[4] = c2.x; s[5] = c2.y; s[6] = d2.x; s[7] = d2.y;
  };
  for (int row = blockIdx.x; row < p.rows; row += gridDim.x) {
    float ss = 0.f;
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
      const long long off = (long long)row * p.ld + v * 8;
      float s[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      if (p.mc) {
        const uint4 u = multimem_sum_bf16x8(p.mc + off);
        const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        s[0] = a.x; s[1] = a.y; s[2] = b.x; s[3] = b.y; s[4] = c.x; s[5] = c.y; s[6] = d.x; s[7] = d.y;
      } else {
        // issue every peer's load before using any of them: one NVLink round trip instead of `world`
        uint4 u[AR_MAX_WORLD];
#pragma unroll
        for (int r = 0; r < AR_MAX_WORLD; ++r)
          if (r < p.world) u[r] = ld_peer_16(p.peer[(p.rank + r) % p.world] + off);  // start at self, rotate
#pragma unroll
        for (int r = 0; r < AR_MAX_WORLD; ++r)
          if (r < p.world) {
            const float2 a = unpack_bf16x2(u[r].x), b = unpack_bf16x2(u[r].y), c = unpack_bf16x2(u[r].z), d = unpack_bf16x2(u[r].w);
            s[0] += a.x; s[1] += a.y; s[2] += b.x; s[3] += b.y; s[4] += c.x; s[5] += c.y; s[6] += d.x; s[7] += d.y;
          }
      }
      if (p.bias) {
        const uint4 u = *reinterpret_cast<const uint4*>(p.bias + v * 8);
        const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        s[0] += a.x; s[1] += a.y; s[2] += b.x; s[3] += b.y; s[4] += c.x; s[5] += c.y; s[6] += d.x; s[7] += d.y;
      }
      if (p.resid && !p.post_weight) add_resid_store(row, v, s);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        rowbuf[v * 8 + j] = s[j];
        ss += s[j] * s[j];
      }
    }
    if (p.post_weight) {
      // sandwich: branch <- rms_norm(branch) * w_post, then residual += branch
      const float pscale = rsqrtf(block_total(ss) / (float)p.n + p.post_eps);
      ss = 0.f;
      for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
        const uint4 u = *reinterpret_cast<const uint4*>(p.post_weight + v * 8);
        const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        const float w8[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
        float s[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j] = rowbuf[v * 8 + j] * pscale * (p.centered ? 1.f + w8[j] : w8[j]);
        if (p.resid) add_resid_store(row, v, s);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
          rowbuf[v * 8 + j] = s[j];
          ss += s[j] * s[j];
        }
      }
    }
    float scale = 1.f;
    if (p.norm_weight) scale = rsqrtf(block_total(ss) / (float)p.n + p.eps);
    for (int v = threadIdx.x; v < vecs; v += blockDim.x) {
      float s[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) s[j] = rowbuf[v * 8 + j] * scale;  // each thread re-reads what it wrote
      if (p.norm_weight) {
        const uint4 u = *reinterpret_cast<const uint4*>(p.norm_weight + v * 8);
        const float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
        const float w8[8] = {a.x, a.y, b.x, b.y, c.x, c.y, d.x, d.y};
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j] *= p.centered ? 1.f + w8[j] : w8[j];
      }
      uint4 o;
      o.x = pack_bf16x2(s[0], s[1]); o.y = pack_bf16x2(s[2], s[3]); o.z = pack_bf16x2(s[4], s[5]); o.w = pack_bf16x2(s[6], s[7]);
      *reinterpret_cast<uint4*>(p.out + (long long)row * p.ld_out + v * 8) = o;
    }
    __syncthreads();
  }

  // "done reading": the last CTA of this rank tells every peer; ticket lives at ctrl[16]. The barrier orders every
  // thread's loads before thread 0's ticket; the release stores order them before the peers' view of the flag.
  if (tracer) p.trace[3] = global_timer_ns();
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence();
    const int t = atomicAdd(p.ctrl + 16, 1);
    if (t == (int)gridDim.x - 1) {
      p.ctrl[16] = 0;
      ar_fence_release_sys();
      for (int r = 0; r < p.world; ++r) ar_st_relaxed_sys(p.peer_ctrl[r] + 8 + p.rank, epoch);
    }
    if (tracer) p.trace[4] = global_timer_ns();
  }
}

// Blocks the stream until every peer has finished reading this rank's buffer for `epoch`.
__global__ void allreduce_wait_readers_kernel(const int* ctrl, int world, int epoch, const int* epoch_dev, int* status) {
  if (threadIdx.x == 0) ar_wait_all(ctrl + 8, world, epoch + (epoch_dev ? *epoch_dev : 0), status);
}

}  // namespace nfn

using namespace nfn;

extern "C" int nfn_allreduce_sandwich_norm(const void* const* peer_bufs, const void* multicast_buf, int* ctrl_local, int* const* ctrl_peer,
                                           int rank, int world, int epoch, const int* epoch_dev, int rows, int n, int ld,
                                           const void* bias, const void* post_weight, float post_eps, void* resid, int ld_resid,
                                           const void* norm_weight, float eps, int centered, void* out, int ld_out, nfn_stream_t stream);

static unsigned long long* g_ar_trace = nullptr;
// Debug aid: five device-side timestamps (ns) of CTA 0 of every following launch go to `dev_u64_5` (null switches it off).
extern "C" int nfn_allreduce_set_trace(void* dev_u64_5) {
  g_ar_trace = static_cast<unsigned long long*>(dev_u64_5);
  return 0;
}

extern "C" int nfn_allreduce_resid_norm(const void* const* peer_bufs, const void* multicast_buf, int* ctrl_local, int* const* ctrl_peer,
                                        int rank, int world, int epoch, const int* epoch_dev, int rows, int n, int ld,
                                        const void* bias, void* resid, int ld_resid, const void* norm_weight, float eps,
                                        int centered, void* out, int ld_out, nfn_stream_t stream) {
  return nfn_allreduce_sandwich_norm(peer_bufs, multicast_buf, ctrl_local, ctrl_peer, rank, world, epoch, epoch_dev, rows, n, ld, bias,
                                     nullptr, 0.f, resid, ld_resid, norm_weight, eps, centered, out, ld_out, stream);
}

// As nfn_allreduce_resid_norm; with `post_weight` the reduced rows are RMS-normalised (post_eps, same
// centering) before they are added to the residual stream, as sandwich-norm blocks need.
extern "C" int nfn_allreduce_sandwich_norm(const void* const* peer_bufs, const void* multicast_buf, int* ctrl_local, int* const* ctrl_peer,
                                           int rank, int world, int epoch, const int* epoch_dev, int rows, int n, int ld,
                                           const void* bias, const void* post_weight, float post_eps, void* resid, int ld_resid,
                                           const void* norm_weight, float eps, int centered, void* out, int ld_out, nfn_stream_t stream) {
  if (rows <= 0) return 0;
  if (!peer_bufs || !ctrl_local || !ctrl_peer || !out) return fail(-1, "allreduce_resid_norm: null operand");
  if (world < 1 || world > AR_MAX_WORLD || rank < 0 || rank >= world) return fail(-1, "allreduce_resid_norm: bad rank / world");
  if (n <= 0 || (n & 7) || (ld & 7) || (ld_out & 7) || (resid && (ld_resid & 7))) return fail(-1, "allreduce_resid_norm: N and strides must be multiples of 8");
  if ((size_t)n * 4 > 200 * 1024) return fail(-1, "allreduce_resid_norm: row too wide for the shared-memory row buffer (N <= 51200)");
  ArParams p{};
  for (int r = 0; r < world; ++r) {
    if (!peer_bufs[r] || !ctrl_peer[r]) return fail(-1, "allreduce_resid_norm: missing peer pointer");
    p.peer[r] = static_cast<const __nv_bfloat16*>(peer_bufs[r]);
    p.peer_ctrl[r] = ctrl_peer[r];
  }
  p.mc = static_cast<const __nv_bfloat16*>(multicast_buf);
  p.ctrl = ctrl_local;
  p.rank = rank; p.world = world; p.epoch = epoch; p.epoch_dev = epoch_dev;
  p.rows = rows; p.n = n; p.ld = ld;
  p.bias = static_cast<const __nv_bfloat16*>(bias);
  p.resid = static_cast<__nv_bfloat16*>(resid);
  p.ld_resid = ld_resid;
  p.norm_weight = static_cast<const __nv_bfloat16*>(norm_weight);
  p.eps = eps; p.centered = centered;
  p.post_weight = static_cast<const __nv_bfloat16*>(post_weight);
  p.post_eps = post_eps;
  p.out = static_cast<__nv_bfloat16*>(out);
  p.ld_out = ld_out;
  p.status = status_ptr();
  p.trace = g_ar_trace;
  const size_t smem = (size_t)n * 4;
  if (smem > 48 * 1024 &&
      cudaFuncSetAttribute(allreduce_resid_norm_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024) != cudaSuccess)
    return fail(-2, "allreduce_resid_norm: cannot raise the dynamic shared memory limit");
  const int grid = rows < sm_count() ? rows : sm_count();
  // one 16-byte vector per thread where the row allows it: every remote load of a row is in flight at once
  const int threads = std::min(AR_MAX_THREADS, std::max(256, (n / 8 + 31) / 32 * 32));
  allreduce_resid_norm_kernel<<<grid, threads, smem, static_cast<cudaStream_t>(stream)>>>(p);
  return launch_check("allreduce_resid_norm", 1);
}

extern "C" int nfn_allreduce_wait_readers(const int* ctrl_local, int world, int epoch, const int* epoch_dev, nfn_stream_t stream) {
  if (!ctrl_local || world < 1 || world > AR_MAX_WORLD) return fail(-1, "allreduce_wait_readers: bad arguments");
  allreduce_wait_readers_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(ctrl_local, world, epoch, epoch_dev, status_ptr());
  return launch_check("allreduce_wait_readers", 1);
}
