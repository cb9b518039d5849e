// Per-row LoRA expand for batches in which (almost) every row has its own adapter:
//   y[t, o] += scale[s] * sum_j u[t, m(o)*r_max + j] * B_all[s, o, j],   s = slot[t]
// The tensor-core projection adds the expand as one masked MMA stage per DISTINCT adapter of a token tile, which
// is the right shape when a few adapters serve many rows; when 128 rows bring 128 adapters, each stage multiplies
// a tile that is zero except for one row.  Here the work is laid out by (row, output feature) instead: one thread
// per output feature reads that feature's B row of the token's adapter -- consecutive threads read consecutive
// B rows, i.e. the kernel streams B_all[slot] -- up to the adapter's own rank only, and adds the product to the
// projection's output in place.  Three B layouts are read: row-major [N, out, r_max], the pre-tiled one of
// mlora_pack_lora_b (128-row tiles per 64-wide rank slice, 16-byte chunks XOR-swizzled inside a row), and the
// rank-compact split layout (MLORA_B_SPLIT: rank/8 slices [out, 8] per adapter), whose 16-byte unit per (slice,
// output feature) makes consecutive threads read consecutive memory with no padding in between: DRAM traffic =
// sum over rows of rank * out * 2 bytes, where the padded layouts drag the rest of each 128-byte row along.
#include "linear.cuh"

namespace mlora {
namespace {

constexpr int kExpThreads = 256;
constexpr int kExpMaxRtot = 1024;

__global__ void __launch_bounds__(kExpThreads) lora_expand_rows_kernel(LinearArgs a, int packed) {
  __shared__ float su[kExpMaxRtot];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.y;
  const int o = blockIdx.x * kExpThreads + threadIdx.x;
  const int slot = a.slots[t];
  // MLORA_SILU_MUL (interleaved gate/up rows): the projection left its pre-activations in a.y_in (fp32 [T, out]); every
  // row, with or without adapter, gets its expand added there and leaves as silu(gate) * up in y [T, out / 2].
  const bool silu = (a.flags & MLORA_SILU_MUL) != 0;
  const bool has = slot >= 0 && slot < a.n_adapters;
  if (!has && !silu) return;  // uniform over the CTA
  const int r_tot = a.r_max * a.n_mod;
  if (has) {
    for (int i = threadIdx.x; i < r_tot; i += kExpThreads) su[i] = a.u[(size_t)t * r_tot + i];
  }
  __syncthreads();
  if (o >= a.out) return;  // (SiLU: out is a multiple of 16, so both lanes of a gate/up pair stay or leave)
  // the output element is requested now, with the B row: one round trip for both
  const bool f32 = (a.flags & MLORA_OUT_F32) != 0;
  float* y32 = reinterpret_cast<float*>(a.y) + (size_t)t * a.ldy + o;
  bf16* y16 = reinterpret_cast<bf16*>(a.y) + (size_t)t * a.ldy + o;
  const float y_old = silu ? a.y_in[(size_t)t * a.out + o] : f32 ? *y32 : __bfloat162float(*y16);
  int rank = !has ? 0 : a.full_rank ? a.r_max : a.ranks[slot];
  rank = rank < a.r_max ? rank : a.r_max;
  const float* um = su + module_of(a, o) * a.r_max;
  const int n_chunks = (rank + 7) / 8;
  float acc = 0.f;
  if (packed == 2) {
    // split layout: slice j of this adapter is the [out, 8] block number ranks[n_adapters + slot] + j
    const int first = a.ranks[a.n_adapters + slot];
    const uint4* base = reinterpret_cast<const uint4*>(a.B_all) + (size_t)first * a.out + o;
    for (int c0 = 0; c0 < n_chunks; c0 += 8) {  // up to 8 x 128-bit loads in flight
      uint4 v[8];
#pragma unroll
      for (int c = 0; c < 8; ++c)
        if (c0 + c < n_chunks) v[c] = ld_stream(base + (size_t)(c0 + c) * a.out);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c0 + c < n_chunks) {
          float bf[8];
          unpack8(v[c], bf);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc = fmaf(um[(c0 + c) * 8 + e], bf[e], acc);
        }
      }
    }
  } else if (!packed) {
    const bf16* b = a.B_all + ((size_t)slot * a.out + o) * a.r_max;
    for (int c0 = 0; c0 < n_chunks; c0 += 8) {  // up to 8 x 128-bit loads in flight
      uint4 v[8];
#pragma unroll
      for (int c = 0; c < 8; ++c)
        if (c0 + c < n_chunks) v[c] = ld_stream(b + (c0 + c) * 8);
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c0 + c < n_chunks) {
          float bf[8];
          unpack8(v[c], bf);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc = fmaf(um[(c0 + c) * 8 + e], bf[e], acc);
        }
      }
    }
  } else {
    const int lora_sub = a.r_max < 64 ? a.r_max : 64, n_sub = a.r_max / lora_sub;
    const int chunks = lora_sub / 8, rb = lora_sub * 2;
    const int row_tiles = (a.out + 127) / 128, row_tile = o >> 7, r = o & 127;
    const int sw = rb == 128 ? (r & 7) : rb == 64 ? ((r >> 1) & 3) : ((r >> 2) & 1);
    const uint4* base = reinterpret_cast<const uint4*>(a.B_all) + ((size_t)slot * row_tiles + row_tile) * n_sub * (128 * chunks) +
                        (size_t)r * chunks;
    for (int sb = 0; sb * chunks < n_chunks; ++sb) {
      uint4 v[8];
#pragma unroll
      for (int c = 0; c < 8; ++c)
        if (c < chunks && sb * chunks + c < n_chunks) v[c] = ld_stream(base + (size_t)sb * (128 * chunks) + (c ^ sw));
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        if (c < chunks && sb * chunks + c < n_chunks) {
          float bf[8];
          unpack8(v[c], bf);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc = fmaf(um[(sb * chunks + c) * 8 + e], bf[e], acc);
        }
      }
    }
  }
  const float y_new = has ? fmaf(acc, a.scales[slot], y_old) : y_old;
  if (silu) {
    // rows 16j..16j+7 are gate, 16j+8..16j+15 the matching up rows: lane pairs 8 apart
    const float other = __shfl_xor_sync(__activemask(), y_new, 8);
    if ((o & 8) == 0)
      reinterpret_cast<bf16*>(a.y)[(size_t)t * a.ldy + (o >> 4) * 8 + (o & 7)] = __float2bfloat16_rn(silu_mul(y_new, other));
    return;
  }
  if (f32)
    *y32 = y_new;
  else
    *y16 = __float2bfloat16_rn(y_new);
}

}  // namespace

bool lora_expand_rows_supported(const LinearArgs& a) {
  if ((a.flags & MLORA_B_SPLIT) && ((a.flags & MLORA_B_PACKED) || a.full_rank)) return false;
  return a.u != nullptr && !(a.flags & MLORA_SILU_MUL) && a.r_max % 8 == 0 && a.r_max * a.n_mod <= kExpMaxRtot &&
         (!(a.flags & MLORA_B_PACKED) || a.r_max == 16 || a.r_max == 32 || a.r_max == 64 || a.r_max == 128) && a.T <= 65535;
}

bool lora_expand_silu_supported(const LinearArgs& a) {
  return a.u != nullptr && (a.flags & MLORA_SILU_MUL) && !(a.flags & (MLORA_B_SPLIT | MLORA_OUT_F32)) && a.out % 16 == 0 &&
         a.r_max % 8 == 0 && a.r_max * a.n_mod <= kExpMaxRtot &&
         (!(a.flags & MLORA_B_PACKED) || a.r_max == 16 || a.r_max == 32 || a.r_max == 64 || a.r_max == 128) && a.T <= 65535;
}

int launch_lora_expand_rows(const LinearArgs& a, cudaStream_t st) {
  dim3 grid((a.out + kExpThreads - 1) / kExpThreads, a.T);
  launch_pdl_if(pdl_enabled(), lora_expand_rows_kernel, grid, dim3(kExpThreads), 0, st, a,
                (a.flags & MLORA_B_SPLIT) ? 2 : (a.flags & MLORA_B_PACKED) ? 1 : 0);
  count_launch();
  MLORA_CHECK_LAUNCH("lora_expand_rows_kernel");
  return MLORA_OK;
}

}  // namespace mlora
