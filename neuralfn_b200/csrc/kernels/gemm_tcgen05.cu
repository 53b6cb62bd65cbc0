// Host side of the BF16 GEMM family: argument validation, tile-shape and split-K
// selection, TMA descriptor set-up and launch. The device code is in gemm_kernel.cuh.
//
// Either operand may be K-major or MN-major, which gives the forward (X W^T),
// input-gradient (dY W) and weight-gradient (dY^T X) products without any transpose
// in memory. Weight-gradient shapes (small M x N output, very long K) are split along
// K into fp32 partial slices that a second small kernel sums.
//
// Covers the role of the reference's linear kernels and library GEMM call sites
// (neuralfn/csrc/tile_cuda/kernels.cu:16746-17574 and its cuBLASLt wrappers) with
// the bias / GELU / residual / dGELU / accumulate epilogues fused.
#include "gemm_kernel.cuh"

namespace nfn {

// out[m, n] = alpha * sum_s part[s][m][n] (+ out when accumulate); bf16 or fp32 output
__global__ void __launch_bounds__(256)
splitk_reduce_kernel(const float* __restrict__ part, long long slice, int splits, void* out, int ldc,
                     int m, int n, float alpha, int out_f32, int accumulate) {
  const int vec_per_row = n / 8;
  const long long idx = (long long)blockIdx.x * 256 + threadIdx.x;
  if (idx >= (long long)m * vec_per_row) return;
  const int row = (int)(idx / vec_per_row), col = (int)(idx % vec_per_row) * 8;
  float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
  for (int s = 0; s < splits; ++s) {
    const float* p = part + (size_t)s * slice + (size_t)row * n + col;
    const float4 a = reinterpret_cast<const float4*>(p)[0], b = reinterpret_cast<const float4*>(p)[1];
    v[0] += a.x; v[1] += a.y; v[2] += a.z; v[3] += a.w;
    v[4] += b.x; v[5] += b.y; v[6] += b.z; v[7] += b.w;
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) v[j] *= alpha;
  if (out_f32) {
    float* cp = static_cast<float*>(out) + (size_t)row * ldc + col;
    if (accumulate) {
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += cp[j];
    }
    reinterpret_cast<float4*>(cp)[0] = make_float4(v[0], v[1], v[2], v[3]);
    reinterpret_cast<float4*>(cp)[1] = make_float4(v[4], v[5], v[6], v[7]);
  } else {
    __nv_bfloat16* cp = static_cast<__nv_bfloat16*>(out) + (size_t)row * ldc + col;
    if (accumulate) {
      float c8[8];
      unpack8_bf16(*reinterpret_cast<const uint4*>(cp), c8);
#pragma unroll
      for (int j = 0; j < 8; ++j) v[j] += c8[j];
    }
    *reinterpret_cast<uint4*>(cp) = pack8_bf16(v);
  }
}

// bf16 epilogue route: 1 (default) = straight from registers with 32-byte stores, no epilogue-wide
// synchronisation; 0 = shared-memory staging tiles + TMA stores. -1 = read NFN_GEMM_EPI_DIRECT once.
static int g_epi_direct = -1;
int epi_direct_flag() {
  if (g_epi_direct < 0) {
    const char* e = getenv("NFN_GEMM_EPI_DIRECT");
    g_epi_direct = (e && e[0] == '0') ? 0 : 1;
  }
  return g_epi_direct ? NFN_EPI_DIRECT_ST : 0;
}

// group_rows != nullptr: the grouped contraction (GemmParams::group_rows) with `groups` slices of C, group_stride elements apart.
template <int BN, int STAGES, bool A_MN, bool B_MN>
static int launch_gemm(const nfn_gemm_args& a, int split_k, cudaStream_t stream, const int* group_rows = nullptr, int groups = 0,
                       long long group_stride = 0) {
  constexpr size_t SMEM =
      (size_t)STAGES * (BM * BK * 2 + BN * BK * 2) + 2 * EPI_TILE_BYTES + 1024 + 256;
  static bool attr_set[64] = {};
  int dev = 0;
  cudaGetDevice(&dev);
  auto kern = gemm_bf16_kernel<BN, STAGES, A_MN, B_MN>;
  if (!attr_set[dev & 63]) {
    if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM) !=
        cudaSuccess)
      return launch_check("gemm attr", 0);
    attr_set[dev & 63] = true;
  }
  CUtensorMap ta, tb, tc, tx;
  bool ok;
  if (!A_MN) ok = make_tmap_2d(&ta, a.a, 2, (uint64_t)a.k, (uint64_t)a.m, (uint64_t)a.lda, BK, BM, 128);
  else       ok = make_tmap_2d(&ta, a.a, 2, (uint64_t)a.m, (uint64_t)a.k, (uint64_t)a.lda, 64, BK, 128);
  if (!ok) return -3;
  if (!B_MN) ok = make_tmap_2d(&tb, a.b, 2, (uint64_t)a.k, (uint64_t)a.n, (uint64_t)a.ldb, BK, BN, 128);
  else       ok = make_tmap_2d(&tb, a.b, 2, (uint64_t)a.n, (uint64_t)a.k, (uint64_t)a.ldb, 64, BK, 128);
  if (!ok) return -3;

  GemmParams p;
  p.c = a.c;
  p.bias = static_cast<const __nv_bfloat16*>(a.bias);
  p.aux_in = static_cast<const __nv_bfloat16*>(a.aux_in);
  p.aux_out = static_cast<__nv_bfloat16*>(a.aux_out);
  p.m = a.m; p.n = a.n; p.k = a.k;
  p.ldc = a.ldc; p.ld_aux_in = a.ld_aux_in; p.ld_aux_out = a.ld_aux_out;
  p.flags = a.flags | epi_direct_flag(); p.alpha = a.alpha; p.act_param = a.act_param;
  p.tiles_m = ceil_div(a.m, BM);
  p.tiles_n = ceil_div(a.n, BN);
  p.split_k = 1;
  p.kb_per_split = ceil_div(a.k, BK);
  p.split_stride = 0;
  p.status = status_ptr();
  p.raster_gw = A_MN ? 1 : pick_raster_gw(a.m, a.k, p.tiles_n);

  const bool out_f32 = a.flags & NFN_EPI_OUT_F32;
  const bool accum = a.flags & NFN_EPI_ACCUM;
  if (group_rows) {
    p.group_rows = group_rows;
    p.split_k = groups;
    p.split_stride = group_stride;
    p.flags |= NFN_EPI_DIRECT_ST;
    p.raster_gw = 1;
    split_k = 1;
    tc = ta; tx = ta;  // direct stores only
  } else if (split_k > 1) {
    // partial products go to fp32 slices of the workspace; the reduce kernel finishes
    p.kb_per_split = ceil_div(ceil_div(a.k, BK), split_k);
    split_k = ceil_div(ceil_div(a.k, BK), p.kb_per_split);  // no empty trailing slice
    p.split_k = split_k;
    p.split_stride = (long long)a.m * a.n;
    p.c = a.workspace;
    p.ldc = a.n;
    p.flags = NFN_EPI_OUT_F32;
    p.alpha = 1.f;
    tc = ta; tx = ta;  // unused on this path
  } else if (!out_f32 && !accum) {
    if (!make_tmap_2d(&tc, a.c, 2, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ldc, EPI_CHUNK, BM, 128))
      return -3;
    if (a.flags & NFN_EPI_SAVE_PRE) {
      if (!make_tmap_2d(&tx, a.aux_out, 2, (uint64_t)a.n, (uint64_t)a.m, (uint64_t)a.ld_aux_out,
                        EPI_CHUNK, BM, 128))
        return -3;
    } else {
      tx = tc;
    }
  } else {
    tc = ta; tx = ta;
  }
  const int tiles = p.tiles_m * p.tiles_n * p.split_k;
  const int grid = tiles < sm_count() ? tiles : sm_count();
  kern<<<grid, GEMM_THREADS, SMEM, stream>>>(ta, tb, tc, tx, p);
  int launched = 1;
  if (split_k > 1) {
    const long long total = (long long)a.m * (a.n / 8);
    splitk_reduce_kernel<<<(unsigned)((total + 255) / 256), 256, 0, stream>>>(
        static_cast<const float*>(a.workspace), (long long)a.m * a.n, split_k, a.c, a.ldc, a.m, a.n,
        a.alpha, out_f32 ? 1 : 0, accum ? 1 : 0);
    launched = 2;
  }
  return launch_check("gemm", launched);
}

int try_launch_gemm_pair(const nfn_gemm_args& a, cudaStream_t stream);  // gemm_2cta.cu

// CTA-pair (cta_group::2) kernel for eligible K-major products: -1 = read NFN_GEMM_PAIR once.
static int g_pair_mode = -1;
int try_launch_gemv(const nfn_gemm_args& a, cudaStream_t stream);  // gemv_bf16.cu
int try_launch_skinny(const nfn_gemm_args& a, cudaStream_t stream);  // gemm_skinny.cu
static int g_gemv_mode = 1;
static int gemv_mode() { return g_gemv_mode; }

static bool pair_enabled() {
  if (g_pair_mode < 0) {
    const char* e = getenv("NFN_GEMM_PAIR");
    g_pair_mode = (e && e[0] == '0') ? 0 : 1;  // on unless NFN_GEMM_PAIR=0
  }
  return g_pair_mode == 1;
}

}  // namespace nfn

// 1 (default): products with at most two rows go to the streaming GEMV kernel; 0: always the tensor-core path.
extern "C" int nfn_gemm_set_gemv_mode(int on) {
  const int old = nfn::g_gemv_mode;
  nfn::g_gemv_mode = on ? 1 : 0;
  return old;
}

extern "C" int nfn_gemm_set_epilogue_direct(int on) {
  const int old = nfn::epi_direct_flag() ? 1 : 0;
  nfn::g_epi_direct = on ? 1 : 0;
  return old;
}

extern "C" int nfn_gemm_set_pair_mode(int on) {
  const int old = nfn::pair_enabled() ? 1 : 0;
  nfn::g_pair_mode = on ? 1 : 0;
  return old;
}

// Grouped contraction: C[g] (M x N, group_stride elements apart, bf16 or fp32) = alpha * A[rows of g]^T-style product over the
// K rows [group_rows[g], group_rows[g + 1]) only. A and B are MN-major ([K, M] and [K, N]: the activations and the upstream
// gradients of an expert-sorted token buffer), group_rows holds groups + 1 row offsets on the device, multiples of 64; rows
// between a group's last real row and the next offset must be finite in both operands and zero in at least one (the MoE plan
// pads segments with zero rows). One launch for all groups, no host read of the counts; a group without rows gives zeros.
// Flags: alpha, fp32 output and accumulate are honoured; there is no bias / activation / residual here.
extern "C" int nfn_gemm_grouped_k(const nfn_gemm_args* args, const int* group_rows, int groups, long long group_stride, nfn_stream_t stream_) {
  using namespace nfn;
  if (!args || !group_rows || groups <= 0) return fail(-1, "gemm_grouped_k: bad arguments");
  const nfn_gemm_args& a = *args;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a.m <= 0 || a.n <= 0 || a.k <= 0) return fail(-1, "gemm_grouped_k: empty problem");
  if (!a.a_mn || !a.b_mn) return fail(-1, "gemm_grouped_k: both operands must be MN-major ([K, M] and [K, N])");
  if ((a.m & 7) || (a.n & 7) || (a.ldc & 7) || (a.lda & 7) || (a.ldb & 7) || (group_stride & 7))
    return fail(-1, "gemm_grouped_k: M, N, leading dimensions and the group stride must be multiples of 8");
  if ((reinterpret_cast<uintptr_t>(a.a) | reinterpret_cast<uintptr_t>(a.b) | reinterpret_cast<uintptr_t>(a.c)) & 15)
    return fail(-1, "gemm_grouped_k: operands must be 16-byte aligned");
  if (a.flags & ~(NFN_EPI_OUT_F32 | NFN_EPI_ACCUM)) return fail(-1, "gemm_grouped_k: only fp32 output and accumulate are supported");
  const int tiles256 = ceil_div(a.m, BM) * ceil_div(a.n, 256) * groups;
  if (tiles256 >= sm_count() && (a.n % 256 == 0 || a.n >= 1024)) return launch_gemm<256, 4, true, true>(a, 1, stream, group_rows, groups, group_stride);
  return launch_gemm<128, 6, true, true>(a, 1, stream, group_rows, groups, group_stride);
}

extern "C" int nfn_gemm_bf16(const nfn_gemm_args* args, nfn_stream_t stream_) {
  using namespace nfn;
  if (!args) return fail(-1, "null args");
  const nfn_gemm_args& a = *args;
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a.m <= 0 || a.n <= 0 || a.k <= 0) return fail(-1, "gemm: empty problem");
  if ((a.n & 7) || (a.ldc & 7)) return fail(-1, "gemm: N and ldc must be multiples of 8");
  if ((a.lda & 7) || (a.ldb & 7)) return fail(-1, "gemm: lda/ldb must be multiples of 8");
  if ((reinterpret_cast<uintptr_t>(a.a) | reinterpret_cast<uintptr_t>(a.b) |
       reinterpret_cast<uintptr_t>(a.c)) & 15)
    return fail(-1, "gemm: operands must be 16-byte aligned");
  if ((a.flags & NFN_EPI_BIAS) && !a.bias) return fail(-1, "gemm: bias flag without bias");
  if ((a.flags & (NFN_EPI_RESID | NFN_EPI_DACT)) && (!a.aux_in || (a.ld_aux_in & 7)))
    return fail(-1, "gemm: aux_in missing or misaligned");
  if ((a.flags & NFN_EPI_RESID) && (a.flags & NFN_EPI_DACT))
    return fail(-1, "gemm: RESID and DACT both read aux_in");
  if ((a.flags & NFN_EPI_SAVE_PRE) &&
      (!a.aux_out || (a.ld_aux_out & 7) || (reinterpret_cast<uintptr_t>(a.aux_out) & 15)))
    return fail(-1, "gemm: aux_out missing or misaligned");

  if (a.m <= 2 && gemv_mode() != 0) {  // one or two rows: pure weight streaming (gemv_bf16.cu)
    const int rc = try_launch_gemv(a, stream);
    if (rc != 0) return rc < 0 ? rc : 0;
  }
  if (a.m >= 3 && a.m <= 64) {  // a handful of rows over a large weight matrix: mma.sync weight streaming (gemm_skinny.cu)
    const int rc = try_launch_skinny(a, stream);
    if (rc != 0) return rc < 0 ? rc : 0;
  }
  const int sms = sm_count();
  const int tiles256 = ceil_div(a.m, BM) * ceil_div(a.n, 256);
  const bool wide = tiles256 >= sms && (a.n % 256 == 0 || a.n >= 1024);
  // split-K: only for plain products (no fused element-wise epilogue) that leave most
  // SMs idle while K is long - the weight-gradient shapes
  int split = 1;
  const int plain_mask = NFN_EPI_BIAS | NFN_EPI_SAVE_PRE | NFN_EPI_RESID | NFN_EPI_DACT | (0xF << NFN_EPI_ACT_SHIFT);
  if (a.split_k > 1 || a.split_k == 0) {
    const int tiles = wide ? tiles256 : ceil_div(a.m, BM) * ceil_div(a.n, 128);
    const int kb = ceil_div(a.k, BK);
    int want = a.split_k > 1 ? a.split_k : 1;
    if (a.split_k == 0 && a.m <= BM && kb >= 16) {
      // one row tile (decode / verification: M = batch): the product only streams the weights and
      // is bound by HBM, so what matters is that every SM streams the same share. Pick the
      // k-blocks per slice that minimise waves x (slice length + per-tile overhead), with the
      // fp32 partial slices kept below about a tenth of the weight bytes.
      const int overhead_kb = 2;
      const long long max_split = std::max(1LL, (long long)a.k / (20LL * a.m));
      long long best_cost = -1;
      for (int per = kb; per >= 2; --per) {
        const int s = ceil_div(kb, per);
        if (s > max_split || s > 64) break;
        const long long waves = ((long long)tiles * s + sms - 1) / sms;
        const long long cost = waves * (per + overhead_kb);
        if (best_cost < 0 || cost < best_cost) { best_cost = cost; want = s; }
      }
    } else if (a.split_k == 0 && tiles * 2 <= sms && kb >= 32) {
      want = sms / tiles;
      if (want > 16) want = 16;
      if (want > kb / 8) want = kb / 8;
    }
    if (want > 1 && !(a.flags & plain_mask) && a.workspace &&
        (long long)want * a.m * a.n * 4 <= a.workspace_bytes)
      split = want;
  }
  if (wide && split == 1 && !a.a_mn && pair_enabled()) {
    const int rc = try_launch_gemm_pair(a, stream);
    if (rc != 0) return rc < 0 ? rc : 0;
  }
#define NFN_DISPATCH(AMN, BMN)                                              \
  return wide ? launch_gemm<256, 4, AMN, BMN>(a, split, stream)             \
              : launch_gemm<128, 6, AMN, BMN>(a, split, stream)
  if (!a.a_mn && !a.b_mn) { NFN_DISPATCH(false, false); }
  if (!a.a_mn && a.b_mn) { NFN_DISPATCH(false, true); }
  if (a.a_mn && !a.b_mn) { NFN_DISPATCH(true, false); }
  NFN_DISPATCH(true, true);
#undef NFN_DISPATCH
}
