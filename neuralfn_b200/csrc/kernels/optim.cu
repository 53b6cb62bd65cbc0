// Optimizer kernels.
//
// Single GPU: squared-norm partials over the flat bf16 gradient, clip factor kept
// on the device, and one AdamW launch over the flat parameter space (fp32 master,
// m, v; bf16 shadow written in the same pass).
//
// Data parallel (one process per GPU, peers mapped through symmetric memory): the
// gradient reduce-scatter, the bf16->fp32 cast/scale, the sharded AdamW update and
// the parameter all-gather are done by two kernels that read the peers' gradient
// buffers and write the peers' parameter buffers directly over NVLink:
//
//   arrive/wait "grads ready"  ->  dp_reduce (peer loads, fp32 shard + sumsq partials)
//   -> publish/collect squared norms (peer stores; doubles as "reads finished" barrier)
//   -> dp_adamw (update owned shard, store bf16 params into every peer)
//   -> arrive/wait "params ready"
//
// Signals are monotonically increasing epochs written with st.release.sys and
// polled with ld.acquire.sys; every wait is bounded by wall-clock time and reports
// NFN_ERR_WAIT_PEER through the status word instead of spinning forever. Arrive and
// wait are separate launches so that a single-GPU emulation can run all "ranks"
// arrive phases before any wait phase.
//
// Reference counterparts: sumsq_partials / global_norm_clip_scale / adamw_step_many*
// (neuralfn/csrc/tile_cuda/kernels.cu:11614-12137); the collective part has no
// counterpart there (the reference has no data parallelism).
#include "common.h"
#include "sm100_ptx.cuh"

namespace nfn {

constexpr int MAX_PEERS = 16;
struct PeerTable {
  void* p[MAX_PEERS];
};

// hyper-parameter block (device fp32[16]) so captured graphs see per-step values
enum { HP_LR = 0, HP_BETA1, HP_BETA2, HP_EPS, HP_WD, HP_BC1, HP_BC2, HP_GRAD_SCALE, HP_MAX_NORM };

__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float block_sum_256(float v, float* red) {
  v = warp_sum_f(v);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
  __syncthreads();
  float t = 0.f;
  if (threadIdx.x < 32) {
    t = threadIdx.x < 8 ? red[threadIdx.x] : 0.f;
    t = warp_sum_f(t);
  }
  return t;  // valid on thread 0
}

__device__ __forceinline__ void unpack8(const uint4& u, float (&f)[8]) {
  float2 a = unpack_bf16x2(u.x), b = unpack_bf16x2(u.y), c = unpack_bf16x2(u.z), d = unpack_bf16x2(u.w);
  f[0] = a.x; f[1] = a.y; f[2] = b.x; f[3] = b.y; f[4] = c.x; f[5] = c.y; f[6] = d.x; f[7] = d.y;
}

// ------------------------------------------------------------ grad norm ------
__global__ void __launch_bounds__(256)
sumsq_bf16_kernel(const __nv_bfloat16* __restrict__ g, long long n8, float* __restrict__ partial) {
  __shared__ float red[8];
  float s = 0.f;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n8; i += (long long)gridDim.x * 256) {
    float f[8];
    unpack8(reinterpret_cast<const uint4*>(g)[i], f);
#pragma unroll
    for (int j = 0; j < 8; ++j) s += f[j] * f[j];
  }
  s = block_sum_256(s, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = s;
}

// clip[0] = min(1, max_norm / (norm + 1e-6)) (1 when max_norm <= 0), clip[1] = norm.
// The squared norm is scaled by grad_scale^2 first (grads are stored unscaled).
__global__ void __launch_bounds__(256)
clip_scale_kernel(const float* __restrict__ partial, int n, const float* __restrict__ hyper,
                  float* __restrict__ clip) {
  __shared__ float red[8];
  float s = 0.f;
  for (int i = threadIdx.x; i < n; i += 256) s += partial[i];
  s = block_sum_256(s, red);
  if (threadIdx.x == 0) {
    const float gs = hyper[HP_GRAD_SCALE];
    const float norm = sqrtf(s) * gs;
    const float mx = hyper[HP_MAX_NORM];
    clip[0] = (mx > 0.f && norm > mx) ? mx / (norm + 1e-6f) : 1.f;
    clip[1] = norm;
  }
}

// ---------------------------------------------------------------- AdamW ------
template <bool GRAD_F32, int NPEERS_OUT>
__device__ __forceinline__ void adamw_vec8(float (&w)[8], float (&m)[8], float (&v)[8],
                                           const float (&g)[8], float lr, float b1, float b2,
                                           float eps, float wd, float bc1, float bc2) {
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    m[j] = b1 * m[j] + (1.f - b1) * g[j];
    v[j] = b2 * v[j] + (1.f - b2) * g[j] * g[j];
    const float mh = m[j] / bc1, vh = v[j] / bc2;
    w[j] -= lr * (mh / (sqrtf(vh) + eps) + wd * w[j]);
  }
}

__device__ __forceinline__ void ld8f(const float* p, float (&f)[8]) {
  const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
  f[0] = a.x; f[1] = a.y; f[2] = a.z; f[3] = a.w; f[4] = b.x; f[5] = b.y; f[6] = b.z; f[7] = b.w;
}
__device__ __forceinline__ void st8f(float* p, const float (&f)[8]) {
  reinterpret_cast<float4*>(p)[0] = make_float4(f[0], f[1], f[2], f[3]);
  reinterpret_cast<float4*>(p)[1] = make_float4(f[4], f[5], f[6], f[7]);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
  uint4 u;
  u.x = pack_bf16x2(f[0], f[1]); u.y = pack_bf16x2(f[2], f[3]);
  u.z = pack_bf16x2(f[4], f[5]); u.w = pack_bf16x2(f[6], f[7]);
  return u;
}

// flat AdamW: elements [0, n_decay) get weight decay. n, n_decay multiples of 8.
__global__ void __launch_bounds__(256)
adamw_flat_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                  const __nv_bfloat16* __restrict__ grad, __nv_bfloat16* __restrict__ param,
                  long long n8, long long decay8, const float* __restrict__ hyper,
                  const float* __restrict__ clip) {
  const float lr = hyper[HP_LR], b1 = hyper[HP_BETA1], b2 = hyper[HP_BETA2], eps = hyper[HP_EPS];
  const float wd = hyper[HP_WD], bc1 = hyper[HP_BC1], bc2 = hyper[HP_BC2];
  const float gscale = hyper[HP_GRAD_SCALE] * (clip ? clip[0] : 1.f);
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n8; i += (long long)gridDim.x * 256) {
    float g[8], w[8], mm[8], vv[8];
    unpack8(reinterpret_cast<const uint4*>(grad)[i], g);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= gscale;
    ld8f(master + i * 8, w); ld8f(m + i * 8, mm); ld8f(v + i * 8, vv);
    adamw_vec8<false, 0>(w, mm, vv, g, lr, b1, b2, eps, i < decay8 ? wd : 0.f, bc1, bc2);
    st8f(master + i * 8, w); st8f(m + i * 8, mm); st8f(v + i * 8, vv);
    reinterpret_cast<uint4*>(param)[i] = pack8(w);
  }
}

// ---------------------------------------------------------- peer signals ------
__device__ __forceinline__ void st_release_sys(int* p, int v) {
  asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int ld_acquire_sys(const int* p) {
  int v;
  asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
__device__ __forceinline__ unsigned long long globaltimer_ns() { return global_timer_ns(); }
// Wait until *p >= want. Returns false on timeout.
__device__ __forceinline__ bool wait_flag_ge(const int* p, int want, unsigned long long timeout_ns) {
  const unsigned long long t0 = globaltimer_ns();
  for (;;) {
    if (ld_acquire_sys(p) >= want) return true;
    __nanosleep(200);
    if (globaltimer_ns() - t0 > timeout_ns) return false;
  }
}

// flags layout on every rank: int[slots][world]. Rank r signals slot s by writing
// `epoch` into every peer's flags[s][r].
__global__ void peer_arrive_kernel(PeerTable flags, int rank, int world, int slot, int epoch,
                                   const int* epoch_dev) {
  if (epoch_dev) epoch += *epoch_dev;
  __threadfence_system();
  const int t = threadIdx.x;
  if (t < world) st_release_sys(static_cast<int*>(flags.p[t]) + slot * world + rank, epoch);
}
__global__ void peer_wait_kernel(const int* my_flags, int world, int slot, int epoch, const int* epoch_dev,
                                 unsigned long long timeout_ns, int* status) {
  const int t = threadIdx.x;
  if (epoch_dev) epoch += *epoch_dev;
  if (t < world) {
    if (!wait_flag_ge(my_flags + slot * world + t, epoch, timeout_ns)) atomicCAS(status, 0, NFN_ERR_WAIT_PEER);
  }
  __threadfence_system();
}

// ------------------------------------------------------ DP reduce-scatter ------
// For the owned shard [lo8, lo8 + n8) (in 8-element vectors): sum the bf16 gradients
// of all peers in fp32, store the fp32 shard and per-block squared-norm partials.
__global__ void __launch_bounds__(256)
dp_reduce_kernel(PeerTable grads, int rank, int world, long long lo8, long long n8,
                 float* __restrict__ gshard, float* __restrict__ partial) {
  __shared__ float red[8];
  float ss = 0.f;
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n8; i += (long long)gridDim.x * 256) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    uint4 u[MAX_PEERS];
#pragma unroll
    for (int r = 0; r < MAX_PEERS; ++r) {
      if (r < world) {
        const int peer = (rank + r) % world;  // start at home, stagger peers across ranks
        u[r] = reinterpret_cast<const uint4*>(grads.p[peer])[lo8 + i];
      }
    }
#pragma unroll
    for (int r = 0; r < MAX_PEERS; ++r) {
      if (r < world) {
        float f[8];
        unpack8(u[r], f);
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[j] += f[j];
      }
    }
    st8f(gshard + i * 8, acc);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += acc[j] * acc[j];
  }
  ss = block_sum_256(ss, red);
  if (threadIdx.x == 0) partial[blockIdx.x] = ss;
}

// Bucketed ("relay") form of the reduce, for overlapping the reduction with the backward pass: the
// 8-element vectors [b8, b8 + n8) of the flat space - a bucket of layers whose gradients are final on
// every rank - are split evenly over the ranks regardless of who owns them. This rank sums its slice
// over all peers' bf16 gradients and stores each fp32 sum into the reduced-gradient shard of the rank
// that owns the vector (a peer store unless that is this rank), so all ranks' links are busy for
// every bucket and the optimizer keeps its contiguous shards. Squared-norm partials accumulate over
// the buckets of a step: the norm a rank publishes then covers the vectors it reduced, and the sum
// over ranks is the global norm as before.
//
// THREADS = 128 is the background form: with at most 80 registers a 128-thread block (10 K registers,
// no dynamic shared memory) fits on an SM beside a resident GEMM CTA of the backward pass
// (320 threads x 168 registers), so it neither waits for an SM to drain nor keeps the next GEMM's
// CTA off an SM - a 256-thread block did both and cost more than the overlap saved.
template <int THREADS>
__global__ void __launch_bounds__(THREADS, THREADS == 128 ? 6 : 1)
dp_reduce_relay_kernel(PeerTable grads, PeerTable gshards, int rank, int world, unsigned b8, unsigned n8,
                       unsigned shard8, float* __restrict__ partial, int accumulate) {
  constexpr int INFLIGHT = THREADS == 128 ? 4 : MAX_PEERS;   // loads in flight per thread
  const unsigned per = (n8 + world - 1) / world;
  const unsigned lo = b8 + (unsigned)rank * per;
  unsigned hi = lo + per;
  if (hi > b8 + n8) hi = b8 + n8;
  float ss = 0.f;
  for (unsigned i = lo + blockIdx.x * THREADS + threadIdx.x; i < hi; i += gridDim.x * THREADS) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int r0 = 0; r0 < MAX_PEERS; r0 += INFLIGHT) {
      uint4 u[INFLIGHT];
#pragma unroll
      for (int r = 0; r < INFLIGHT; ++r)
        if (r0 + r < world) u[r] = reinterpret_cast<const uint4*>(grads.p[r0 + r])[i];   // table rotated by the host: entry 0 = this rank
#pragma unroll
      for (int r = 0; r < INFLIGHT; ++r) {
        if (r0 + r < world) {
          float f[8];
          unpack8(u[r], f);
#pragma unroll
          for (int j = 0; j < 8; ++j) acc[j] += f[j];
        }
      }
    }
    const unsigned owner = i / shard8;
    st8f(static_cast<float*>(gshards.p[owner]) + (size_t)(i - owner * shard8) * 8, acc);
#pragma unroll
    for (int j = 0; j < 8; ++j) ss += acc[j] * acc[j];
  }
  // one partial slot per warp: the kernel uses no shared memory at all, so that a block fits on an SM
  // whose shared memory a GEMM CTA has taken whole
  ss = warp_sum_f(ss);
  if ((threadIdx.x & 31) == 0) {
    float* slot = partial + blockIdx.x * (THREADS / 32) + (threadIdx.x >> 5);
    *slot = accumulate ? *slot + ss : ss;
  }
}

// Publish this rank's squared norm (sum of `npartial` partials) into every peer's
// norm slots: slots[rank] = {sumsq, epoch} written as one 8-byte release store.
__global__ void __launch_bounds__(256)
dp_norm_publish_kernel(const float* __restrict__ partial, int npartial, PeerTable norm_slots,
                       int rank, int world, int epoch, const int* epoch_dev) {
  __shared__ float red[8];
  __shared__ float total;
  if (epoch_dev) epoch += *epoch_dev;
  float s = 0.f;
  for (int i = threadIdx.x; i < npartial; i += 256) s += partial[i];
  s = block_sum_256(s, red);
  if (threadIdx.x == 0) total = s;
  __syncthreads();
  __threadfence_system();
  if (threadIdx.x < world) {
    const unsigned long long packed =
        (static_cast<unsigned long long>(static_cast<unsigned>(epoch)) << 32) | __float_as_uint(total);
    unsigned long long* dst = static_cast<unsigned long long*>(norm_slots.p[threadIdx.x]) + rank;
    asm volatile("st.release.sys.global.u64 [%0], %1;" ::"l"(dst), "l"(packed) : "memory");
  }
}
// Wait for all ranks' squared norms of this epoch, then compute the clip factor.
__global__ void dp_norm_collect_kernel(const unsigned long long* my_slots, int world, int epoch,
                                       const int* epoch_dev,
                                       const float* __restrict__ hyper, float* __restrict__ clip,
                                       unsigned long long timeout_ns, int* status) {
  __shared__ float vals[MAX_PEERS];
  __shared__ int bad;
  if (epoch_dev) epoch += *epoch_dev;
  if (threadIdx.x == 0) bad = 0;
  __syncthreads();
  const int t = threadIdx.x;
  if (t < world) {
    const unsigned long long t0 = globaltimer_ns();
    unsigned long long v;
    for (;;) {
      asm volatile("ld.acquire.sys.global.u64 %0, [%1];" : "=l"(v) : "l"(my_slots + t) : "memory");
      if (static_cast<int>(v >> 32) >= epoch) break;
      __nanosleep(200);
      if (globaltimer_ns() - t0 > timeout_ns) { bad = 1; break; }
    }
    vals[t] = __uint_as_float(static_cast<unsigned>(v & 0xffffffffu));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (bad) atomicCAS(status, 0, NFN_ERR_WAIT_PEER);
    float s = 0.f;
    for (int r = 0; r < world; ++r) s += vals[r];
    const float norm = sqrtf(s) * hyper[HP_GRAD_SCALE];
    const float mx = hyper[HP_MAX_NORM];
    clip[0] = (!bad && mx > 0.f && norm > mx) ? mx / (norm + 1e-6f) : 1.f;
    clip[1] = norm;
  }
}

// Sharded AdamW: fp32 reduced gradient shard -> update owned master/m/v -> store the
// bf16 parameters of the shard into every peer's parameter buffer (all-gather by push).
__global__ void __launch_bounds__(256)
dp_adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                const float* __restrict__ gshard, PeerTable params, int rank, int world,
                long long lo8, long long n8, long long decay8_global,
                const float* __restrict__ hyper, const float* __restrict__ clip) {
  const float lr = hyper[HP_LR], b1 = hyper[HP_BETA1], b2 = hyper[HP_BETA2], eps = hyper[HP_EPS];
  const float wd = hyper[HP_WD], bc1 = hyper[HP_BC1], bc2 = hyper[HP_BC2];
  const float gscale = hyper[HP_GRAD_SCALE] * clip[0];
  for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n8; i += (long long)gridDim.x * 256) {
    float g[8], w[8], mm[8], vv[8];
    ld8f(gshard + i * 8, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) g[j] *= gscale;
    ld8f(master + i * 8, w); ld8f(m + i * 8, mm); ld8f(v + i * 8, vv);
    adamw_vec8<true, 0>(w, mm, vv, g, lr, b1, b2, eps, (lo8 + i) < decay8_global ? wd : 0.f, bc1, bc2);
    st8f(master + i * 8, w); st8f(m + i * 8, mm); st8f(v + i * 8, vv);
    const uint4 packed = pack8(w);
#pragma unroll
    for (int r = 0; r < MAX_PEERS; ++r) {
      if (r < world) {
        const int peer = (rank + r) % world;
        reinterpret_cast<uint4*>(params.p[peer])[lo8 + i] = packed;
      }
    }
  }
}

static int grid_for(long long n8) {
  long long blocks = (n8 + 255) / 256;
  const long long cap = (long long)sm_count() * 8;
  return (int)(blocks < 1 ? 1 : (blocks > cap ? cap : blocks));
}

// Kernels that run beside the backward pass on a second stream ask for the largest shared-memory
// carve-out although they use next to none: an SM holds one carve-out at a time and only changes it when
// it is empty, so a block launched with the default (small) carve-out keeps the 227 KB GEMM CTAs off its
// SM until it exits - measured as a GEMM delay equal to the whole side kernel's duration.
static void prefer_max_smem_once() {
  static bool done[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  if (dev < 0 || dev >= 64 || done[dev]) return;
  done[dev] = true;
  cudaFuncSetAttribute(dp_reduce_relay_kernel<128>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  cudaFuncSetAttribute(dp_reduce_relay_kernel<256>, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  cudaFuncSetAttribute(peer_arrive_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
  cudaFuncSetAttribute(peer_wait_kernel, cudaFuncAttributePreferredSharedMemoryCarveout, cudaSharedmemCarveoutMaxShared);
}

static bool fill_table(PeerTable& t, void* const* ptrs, int world) {
  if (world < 1 || world > MAX_PEERS) return false;
  for (int i = 0; i < MAX_PEERS; ++i) t.p[i] = i < world ? ptrs[i] : nullptr;
  return true;
}

}  // namespace nfn

using namespace nfn;

namespace nfn {
__global__ void counter_add_kernel(int* p, int v) { if (threadIdx.x == 0) *p += v; }
}
// *p += v on the stream: the device-resident signal epoch advanced once per step, so a
// captured step graph produces fresh epochs on every replay.
extern "C" int nfn_counter_add(int* p, int v, nfn_stream_t stream) {
  counter_add_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(p, v);
  return launch_check("counter_add");
}

extern "C" int nfn_optim_max_partials(void) { return sm_count() * 8; }

// partial: fp32 [nfn_optim_max_partials()]; clip: fp32 [2]
extern "C" int nfn_grad_clip_scale(const void* grad, long long n, float* partial, const float* hyper,
                                   float* clip, nfn_stream_t stream) {
  if (n % 8) return fail(-1, "grad_clip_scale: n must be a multiple of 8");
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int grid = grid_for(n / 8);
  sumsq_bf16_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)grad, n / 8, partial);
  clip_scale_kernel<<<1, 256, 0, st>>>(partial, grid, hyper, clip);
  return launch_check("grad_clip_scale", 2);
}

extern "C" int nfn_adamw_flat(float* master, float* m, float* v, const void* grad, void* param,
                              long long n, long long n_decay, const float* hyper, const float* clip,
                              nfn_stream_t stream) {
  if (n % 8 || n_decay % 8) return fail(-1, "adamw_flat: n and n_decay must be multiples of 8");
  adamw_flat_kernel<<<grid_for(n / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      master, m, v, (const __nv_bfloat16*)grad, (__nv_bfloat16*)param, n / 8, n_decay / 8, hyper, clip);
  return launch_check("adamw_flat");
}

extern "C" int nfn_peer_arrive(void* const* peer_flags, int rank, int world, int slot, int epoch,
                               const int* epoch_dev,
                               nfn_stream_t stream) {
  PeerTable t;
  if (!fill_table(t, peer_flags, world)) return fail(-1, "peer_arrive: bad world size");
  prefer_max_smem_once();
  peer_arrive_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(t, rank, world, slot, epoch, epoch_dev);
  return launch_check("peer_arrive");
}

extern "C" int nfn_peer_wait(const int* my_flags, int world, int slot, int epoch, const int* epoch_dev,
                             double timeout_s,
                             nfn_stream_t stream) {
  if (world < 1 || world > MAX_PEERS) return fail(-1, "peer_wait: bad world size");
  prefer_max_smem_once();
  peer_wait_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      my_flags, world, slot, epoch, epoch_dev, (unsigned long long)(timeout_s * 1e9), status_ptr());
  return launch_check("peer_wait");
}

// shard = elements [lo, lo + n) of the flat space; lo, n multiples of 8.
extern "C" int nfn_dp_reduce(void* const* peer_grads, int rank, int world, long long lo, long long n,
                             float* gshard, float* partial, nfn_stream_t stream) {
  PeerTable t;
  if (!fill_table(t, peer_grads, world)) return fail(-1, "dp_reduce: bad world size");
  if (lo % 8 || n % 8) return fail(-1, "dp_reduce: shard bounds must be multiples of 8");
  dp_reduce_kernel<<<grid_for(n / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      t, rank, world, lo / 8, n / 8, gshard, partial);
  return launch_check("dp_reduce");
}

// Size of the squared-norm partial array of the bucketed reduce (the largest grid it launches).
extern "C" int nfn_dp_relay_blocks(void) { return sm_count() * 8 * 8; }   // one slot per warp of the largest grid

// Bucket = elements [lo, lo + n) of the flat space (multiples of 8); peer_gshards[r] = rank r's fp32
// reduced-gradient shard of `shard` elements (peer-writable); partial: fp32 [nfn_dp_relay_blocks()],
// zeroed by the caller at the start of a step when `accumulate` is set on every launch.
// `background` != 0: one 128-thread block per SM, for a launch that runs beside the backward pass's
// GEMMs (it is bound by NVLink and must fit next to their CTAs); 0: a full grid, for a launch nothing hides.
extern "C" int nfn_dp_reduce_relay(void* const* peer_grads, void* const* peer_gshards, int rank, int world,
                                   long long lo, long long n, long long shard, float* partial, int accumulate,
                                   int background, nfn_stream_t stream) {
  PeerTable tg, ts;
  if (!fill_table(tg, peer_grads, world) || !fill_table(ts, peer_gshards, world)) return fail(-1, "dp_reduce_relay: bad world size");
  if (lo % 8 || n % 8 || shard % 8 || n < 0 || shard <= 0) return fail(-1, "dp_reduce_relay: bounds must be multiples of 8");
  if (lo < 0 || lo + n > shard * world) return fail(-1, "dp_reduce_relay: bucket outside the flat space");
  if (shard * world / 8 >= (1ll << 31)) return fail(-1, "dp_reduce_relay: flat space too large for 32-bit vector indices");
  prefer_max_smem_once();
  // start at home and stagger the peers across ranks; a fixed order per entry keeps the table in registers
  PeerTable rot = tg;
  for (int r = 0; r < world; ++r) rot.p[r] = tg.p[(rank + r) % world];
  tg = rot;
  const long long slice8 = (n / 8 + world - 1) / world;
  if (background) {
    dp_reduce_relay_kernel<128><<<sm_count(), 128, 0, static_cast<cudaStream_t>(stream)>>>(
        tg, ts, rank, world, (unsigned)(lo / 8), (unsigned)(n / 8), (unsigned)(shard / 8), partial, accumulate);
  } else {
    dp_reduce_relay_kernel<256><<<grid_for(slice8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        tg, ts, rank, world, (unsigned)(lo / 8), (unsigned)(n / 8), (unsigned)(shard / 8), partial, accumulate);
  }
  return launch_check("dp_reduce_relay");
}

// Same as nfn_dp_norm_publish with the number of partials given directly.
extern "C" int nfn_dp_norm_publish_n(const float* partial, int npartial, void* const* peer_slots,
                                     int rank, int world, int epoch, const int* epoch_dev, nfn_stream_t stream) {
  PeerTable t;
  if (!fill_table(t, peer_slots, world)) return fail(-1, "dp_norm_publish: bad world size");
  if (npartial < 1) return fail(-1, "dp_norm_publish: no partials");
  dp_norm_publish_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(partial, npartial, t, rank, world, epoch, epoch_dev);
  return launch_check("dp_norm_publish");
}

extern "C" int nfn_dp_norm_publish(const float* partial, long long shard_n, void* const* peer_slots,
                                   int rank, int world, int epoch, const int* epoch_dev,
                                   nfn_stream_t stream) {
  PeerTable t;
  if (!fill_table(t, peer_slots, world)) return fail(-1, "dp_norm_publish: bad world size");
  dp_norm_publish_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      partial, grid_for(shard_n / 8), t, rank, world, epoch, epoch_dev);
  return launch_check("dp_norm_publish");
}

extern "C" int nfn_dp_norm_collect(const void* my_slots, int world, int epoch, const int* epoch_dev,
                                   const float* hyper,
                                   float* clip, double timeout_s, nfn_stream_t stream) {
  if (world < 1 || world > MAX_PEERS) return fail(-1, "dp_norm_collect: bad world size");
  dp_norm_collect_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(
      (const unsigned long long*)my_slots, world, epoch, epoch_dev, hyper, clip,
      (unsigned long long)(timeout_s * 1e9), status_ptr());
  return launch_check("dp_norm_collect");
}

extern "C" int nfn_dp_adamw(float* master, float* m, float* v, const float* gshard,
                            void* const* peer_params, int rank, int world, long long lo, long long n,
                            long long n_decay_global, const float* hyper, const float* clip,
                            nfn_stream_t stream) {
  PeerTable t;
  if (!fill_table(t, peer_params, world)) return fail(-1, "dp_adamw: bad world size");
  if (lo % 8 || n % 8 || n_decay_global % 8) return fail(-1, "dp_adamw: bounds must be multiples of 8");
  dp_adamw_kernel<<<grid_for(n / 8), 256, 0, static_cast<cudaStream_t>(stream)>>>(
      master, m, v, gshard, t, rank, world, lo / 8, n / 8, n_decay_global / 8, hyper, clip);
  return launch_check("dp_adamw");
}
