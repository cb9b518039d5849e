// CUDA-core kernels of the projection path:
//   * lora_shrink_kernel: u = x . A[slot]^T, one warp per (row, rank index), 128-bit loads,
//     warp-shuffle reduction.
//   * linear_simt_kernel: y = x W^T (+ LoRA expand, + SiLU*up), one warp per output feature,
//     128-bit loads, warp-shuffle reduction.  Shape-agnostic (in % 8 == 0); the small-batch
//     (T <= 8) decode GEMV and the fallback for shapes the tensor-core kernel does not take.
#include "linear.cuh"

namespace mlora {
namespace {

__global__ void __launch_bounds__(256) lora_shrink_kernel(const bf16* __restrict__ x, int64_t ldx,
                                                          const bf16* __restrict__ A_all,
                                                          const int32_t* __restrict__ ranks,
                                                          const int32_t* __restrict__ slots, int n_adapters,
                                                          int in, int r_max, int r_tot, float* __restrict__ u) {
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.y;
  const int j = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  if (j >= r_tot) return;
  const int slot = slots[t];
  float acc = 0.f;
  // Rows of A at or beyond an adapter's rank are zero by contract.  The first 16 rank rows of a module are
  // multiplied without looking the rank up (one dependent global load less in a kernel that is nothing but a chain
  // of round trips: the common rank-16 stacks never pay for it); further rows of wide pitches are skipped when the
  // adapter's own rank is lower, so a rank-8 adapter in a pitch-64 stack does not stream 56 rows of zeros.
  const int jm = j % r_max;
  if (slot >= 0 && slot < n_adapters && (jm < 16 || jm < ranks[slot])) {
    const bf16* a = A_all + ((size_t)slot * r_tot + j) * in;
    const bf16* xr = x + (size_t)t * ldx;
    // 8 chunks of A and of x are requested before the first is used: the dot product is a chain of
    // L2 round trips otherwise (one warp per (row, rank index), nothing else to hide the latency)
    for (int k0 = lane * 8; k0 < in; k0 += 256 * 8) {
      uint4 av[8], xv[8];
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        const int k = k0 + c * 256;
        if (k < in) {
          av[c] = ld_cached(a + k);
          xv[c] = ld_cached(xr + k);
        }
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (k0 + c * 256 < in) {
          float af[8], xf[8];
          unpack8(av[c], af);
          unpack8(xv[c], xf);
#pragma unroll
          for (int i = 0; i < 8; ++i) acc = fmaf(af[i], xf[i], acc);
        }
      }
    }
    acc = warp_sum(acc);
  }
  if (lane == 0) u[(size_t)t * r_tot + j] = acc;
}

template <int TT, bool SILU>
__global__ void __launch_bounds__(256) linear_simt_kernel(LinearArgs a) {
  pdl_launch_dependents();
  pdl_wait();
  const int unit = blockIdx.x * 8 + (threadIdx.x >> 5);
  const int lane = threadIdx.x & 31;
  const int n_units = SILU ? a.out / 2 : a.out;
  if (unit >= n_units) return;
  const int row0 = SILU ? (unit >> 3) * 16 + (unit & 7) : unit;
  const int row1 = row0 + 8;
  const bf16* w0 = a.W + (size_t)row0 * a.in;
  const bf16* w1 = a.W + (size_t)row1 * a.in;
  for (int t0 = 0; t0 < a.T; t0 += TT) {
    float acc0[TT], acc1[TT];
#pragma unroll
    for (int i = 0; i < TT; ++i) acc0[i] = acc1[i] = 0.f;
    for (int k = lane * 8; k < a.in; k += 256) {
      float wf0[8], wf1[8];
      unpack8(ld_cached(w0 + k), wf0);
      if (SILU) unpack8(ld_cached(w1 + k), wf1);
#pragma unroll
      for (int i = 0; i < TT; ++i) {
        if (t0 + i < a.T) {
          float xf[8];
          unpack8(ld_cached(a.x + (size_t)(t0 + i) * a.ldx + k), xf);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            acc0[i] = fmaf(wf0[e], xf[e], acc0[i]);
            if (SILU) acc1[i] = fmaf(wf1[e], xf[e], acc1[i]);
          }
        }
      }
    }
    float v0 = 0.f, v1 = 0.f;
#pragma unroll
    for (int i = 0; i < TT; ++i) {
      float s0 = warp_sum(acc0[i]);
      float s1 = SILU ? warp_sum(acc1[i]) : 0.f;
      if (lane == i) {
        v0 = s0;
        v1 = s1;
      }
    }
    const int t = t0 + lane;
    if (lane < TT && t < a.T) {
      v0 += lora_expand(a, t, row0);
      if (SILU) v1 += lora_expand(a, t, row1);
      store_out(a, t, SILU ? unit : row0, SILU ? silu_mul(v0, v1) : v0);
    }
  }
}

template <int TT>
void launch_simt(const LinearArgs& a, cudaStream_t st) {
  const int n_units = (a.flags & MLORA_SILU_MUL) ? a.out / 2 : a.out;
  const int grid = (n_units + 7) / 8;
  if (a.flags & MLORA_SILU_MUL)
    launch_pdl(linear_simt_kernel<TT, true>, grid, 256, 0, st, a);
  else
    launch_pdl(linear_simt_kernel<TT, false>, grid, 256, 0, st, a);
}

}  // namespace

int launch_linear_simt(const LinearArgs& a, cudaStream_t st) {
  if (a.T <= 1)
    launch_simt<1>(a, st);
  else if (a.T <= 2)
    launch_simt<2>(a, st);
  else if (a.T <= 4)
    launch_simt<4>(a, st);
  else
    launch_simt<8>(a, st);
  count_launch();
  MLORA_CHECK_LAUNCH("linear_simt_kernel");
  return MLORA_OK;
}

}  // namespace mlora

using namespace mlora;

extern "C" int mlora_lora_shrink(const void* d_x, int64_t ldx, const void* d_A_all, const int32_t* d_ranks,
                                 const int32_t* d_slots, int32_t n_adapters, int32_t T, int32_t in, int32_t r_max,
                                 int32_t n_mod, float* d_u, void* stream) {
  MLORA_REQUIRE(T >= 0 && in > 0 && r_max > 0 && n_mod > 0 && n_adapters > 0, "lora_shrink: bad sizes");
  MLORA_REQUIRE(in % 8 == 0 && ldx % 8 == 0, "lora_shrink: in and ldx must be multiples of 8 (in=%d)", in);
  MLORA_REQUIRE(d_x && d_A_all && d_ranks && d_slots && d_u, "lora_shrink: null pointer");
  MLORA_REQUIRE(aligned16(d_x) && aligned16(d_A_all), "lora_shrink: x and A_all must be 16-byte aligned");
  if (T == 0) return MLORA_OK;
  const int r_tot = r_max * n_mod;
  if (lora_shrink_tc_supported(d_x, ldx, d_A_all, d_u, T, in, r_tot))
    return launch_lora_shrink_tc(d_x, ldx, d_A_all, d_slots, n_adapters, T, in, r_tot, d_u, (cudaStream_t)stream);
  MLORA_REQUIRE(T <= 65535, "lora_shrink: T=%d exceeds 65535 rows per call", T);
  dim3 grid((r_tot + 7) / 8, T);
  launch_pdl_if(pdl_enabled_shrink(), lora_shrink_kernel, grid, 256, 0, (cudaStream_t)stream, (const bf16*)d_x, ldx, (const bf16*)d_A_all, d_ranks,
             d_slots, n_adapters, in, r_max, r_tot, d_u);
  count_launch();
  MLORA_CHECK_LAUNCH("lora_shrink_kernel");
  return MLORA_OK;
}
