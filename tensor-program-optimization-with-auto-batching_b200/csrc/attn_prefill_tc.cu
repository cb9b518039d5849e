// Causal attention for prompt rows on the 5th-generation tensor cores (tcgen05 + TMEM): the ragged prefill path of
// paged_kv_cache.attention_with_fused_qkv (tvm/llama_auto_batcher/llama_for_causal_lm.py:55-64, prefill call
// llama_exec_graph.py:75-85) after the rows' keys and values have been appended to the pages.
//
// One CTA = one tile of up to 128 consecutive prompt rows of ONE sequence x one head.  Per block of 128 keys:
//   S = Q K^T      tcgen05.mma, M = 128 queries, N = 128 keys, K = head_dim 128; Q and K both K-major in 128-byte-swizzled
//                  shared memory -- Q by one TMA load per tile, K by one TMA load per page (16 keys) through the block table;
//   softmax        one thread per query row (= TMEM lane): scores read back with tcgen05.ld, causal mask, online maximum
//                  and sum, probabilities written as bf16 into the A-operand layout;
//   O_blk = P V    M = 128 queries, N = 128 head dims, K = 128 keys; V arrives by TMA exactly as the pages hold it,
//                  [key][dim], and is used as an MN-major B operand (the dimension is the contiguous one): no transpose;
//                  P is written over the K block, which S = Q K^T has consumed by then;
//   O = O * exp2(m_old - m_new) + O_blk    in registers (128 fp32 per thread), no read-modify-write of TMEM.
// Inside a CTA the two MMAs of a block and the softmax between them run one after the other; two CTAs share an SM
// (96 KB of shared memory and 256 TMEM columns each) and fill each other's gaps.  The point of this kernel is to take
// prompt attention off the CUDA cores -- the single-query kernel it replaces re-reads every key for every row and
// reduces every score with shuffles.  Every wait is bounded; a CTA that gives up writes zeros.
#include <atomic>

#include "common.cuh"
#include "tc_ptx.cuh"

namespace mlora {
namespace {

constexpr int kD = 128;            // head dimension
constexpr int kPS = 16;            // page size
constexpr int kTile = 128;         // query rows per CTA = keys per block
constexpr int kPfThreads = 160;    // warps 0..3: one thread per query row; warp 4: TMA + MMA issue
constexpr int kSub = kTile * 64 * 2;  // one [128 x 64] bf16 sub-tile: 16 KB
constexpr float kLog2e = 1.4426950408889634f;

__device__ __forceinline__ float fast_exp2(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// Shared-memory descriptor of an MN-major operand tile with 128-byte swizzle: rows of 128 bytes hold 64 consecutive
// M/N elements of one k; `lbo` bytes to the next 64 M/N elements, `sbo` bytes to the next 8 k.
__device__ __forceinline__ uint64_t make_smem_desc_mn(uint32_t saddr, uint32_t lbo, uint32_t sbo) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFFu) >> 4);
  d |= (uint64_t)(lbo >> 4) << 16;
  d |= (uint64_t)(sbo >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

struct PfArgs {
  const int32_t* block_table;
  int max_pages;
  const int32_t* tiles;  // [n_tiles][4]: cache slot, first row (index into qkv / out), rows, position of the first row
  int Hq, Hkv;
  bf16* out;
  int64_t ld_out;
  int32_t* status;  // optional: set to 1 when a wait expired
};

__global__ void __launch_bounds__(kPfThreads, 2) prefill_attn_tc_kernel(const __grid_constant__ CUtensorMap map_q,
                                                                         const __grid_constant__ CUtensorMap map_k,
                                                                         const __grid_constant__ CUtensorMap map_v,
                                                                         PfArgs a) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* sq = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~(uintptr_t)1023);
  uint8_t* sk = sq + 2 * kSub;   // K block   [128 keys][128 d]   as two d-halves
  uint8_t* sv = sk + 2 * kSub;   // V block   [128 keys][128 d]   as two d-halves, exactly as the pages hold it
  uint8_t* sp = sk;              // P block   [128 q][128 keys]   as two key-halves: over K, which S = Q K^T has consumed by then
  __shared__ uint64_t kbar, sbar, obar;
  __shared__ uint32_t tmem_slot;
  __shared__ int s_abort;

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int tile = blockIdx.x, h = blockIdx.y;
  const int rep = a.Hq / a.Hkv, kvh = h / rep;
  const int slot = a.tiles[tile * 4 + 0], row0 = a.tiles[tile * 4 + 1], rows = a.tiles[tile * 4 + 2], pos0 = a.tiles[tile * 4 + 3];
  const int32_t* bt = a.block_table + (size_t)slot * a.max_pages;
  const int n_keys = pos0 + rows;                       // keys any row of the tile may see
  const int n_blocks = (n_keys + kTile - 1) / kTile;
  const int n_pages = (n_keys + kPS - 1) / kPS;

  if (tid == 0) {
    s_abort = 0;
    mbar_init(&kbar, 1);
    mbar_init(&sbar, 1);
    mbar_init(&obar, 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    tma_prefetch_desc(&map_q);
    tma_prefetch_desc(&map_k);
    tma_prefetch_desc(&map_v);
  }
  if (warp == 4) tmem_alloc(&tmem_slot, 256);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = tmem_slot;
  constexpr uint32_t idesc = make_idesc(kTile, kTile);
  constexpr uint32_t idesc_pv = idesc | (1u << 16);  // B operand MN-major

  // per-row state (threads 0..127)
  float o_reg[kD];
#pragma unroll
  for (int i = 0; i < kD; ++i) o_reg[i] = 0.f;
  float m_run = -INFINITY, l_run = 0.f;
  const int q_pos = pos0 + tid;  // position of this thread's query row
  const float scale = rsqrtf((float)kD) * kLog2e;
  bool ok = true;

  // Block-table entries are read one block ahead (lane p of warp 4 keeps page p of the block's eight), so that no block
  // starts with a dependent chain of two global round trips.
  auto page_of = [&](int pg) { return pg < n_pages ? bt[pg] : -1; };
  int page_next = (warp == 4 && lane < kTile / kPS) ? page_of(lane) : -1;

  for (int kb = 0; kb < n_blocks; ++kb) {
    const uint32_t par = kb & 1;
    const int page0 = kb * (kTile / kPS);
    const int page_cur = page_next;
    const int valid = min(kTile / kPS, n_pages - page0);
    if (kb + 1 < n_blocks && warp == 4 && lane < kTile / kPS) page_next = page_of(page0 + kTile / kPS + lane);
    // ---- loads: K and V pages (and Q once) by TMA -----------------------------------------------------------------------------
    if (warp == 4) {
      if (lane == 0) {
        mbar_expect_tx(&kbar, (uint32_t)valid * 4 * (kPS * 128) + (kb == 0 ? 2 * kSub : 0));
        if (kb == 0) {
          tma_load_2d(sq, &map_q, h * kD, row0, &kbar);
          tma_load_2d(sq + kSub, &map_q, h * kD + 64, row0, &kbar);
        }
      }
      __syncwarp();
      if (lane < valid) {  // one page per lane, both 64-column halves of K and of V (a missing table entry reads as rows before 0: zeros)
        const int r = (page_cur * a.Hkv + kvh) * kPS;
        tma_load_2d(sk + lane * (kPS * 128), &map_k, 0, r, &kbar);
        tma_load_2d(sk + kSub + lane * (kPS * 128), &map_k, 64, r, &kbar);
        tma_load_2d(sv + lane * (kPS * 128), &map_v, 0, r, &kbar);
        tma_load_2d(sv + kSub + lane * (kPS * 128), &map_v, 64, r, &kbar);
      }
    } else if (n_keys - kb * kTile < kTile) {
      // Last block, not full: the V rows of keys that do not exist (the tail of the last page, whatever the cache holds
      // there, and the pages that were not loaded) are zeroed once the copies have landed -- their probabilities are 0,
      // but 0 * NaN is not.  K needs nothing: those scores are masked.  (A swizzled row stays inside its own 128 bytes.)
      if (!mbar_wait(&kbar, par, &s_abort)) s_abort = 1;
      if (tid >= n_keys - kb * kTile) {
#pragma unroll
        for (int half = 0; half < 2; ++half)
#pragma unroll
          for (int c = 0; c < 8; ++c) reinterpret_cast<uint4*>(sv + half * kSub + tid * 128)[c] = make_uint4(0u, 0u, 0u, 0u);
      }
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    // ---- S = Q K^T ----------------------------------------------------------------------------------------------------------
    if (tid == 128) {
      if (!mbar_wait(&kbar, par, &s_abort)) s_abort = 1;
      tc_fence_after();
      if (!s_abort) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          const uint64_t adesc = make_smem_desc(smem_u32(sq + j * kSub));
          const uint64_t bdesc = make_smem_desc(smem_u32(sk + j * kSub));
#pragma unroll
          for (int k = 0; k < 4; ++k) umma_bf16(tmem_base, adesc + 2 * k, bdesc + 2 * k, idesc, (j > 0 || k > 0) ? 1u : 0u);
        }
      }
      umma_commit(&sbar);
    }
    float corr = 1.f;
    if (tid < kTile) {
      if (!mbar_wait(&sbar, par, &s_abort)) s_abort = 1;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + ((uint32_t)(warp * 32) << 16);
      // Only the blocks on or past the diagonal need the causal / length mask (uniform per CTA): every row of the
      // tile sees every key of the blocks before.
      const bool need_mask = kb * kTile + kTile - 1 > pos0;
      // pass 1: row maximum over the valid keys (of the raw scores: the scale is positive)
      float mx = -INFINITY;
#pragma unroll 1
      for (int c0 = 0; c0 < kTile; c0 += 32) {
        float s[32];
        tmem_ld32(t_addr + c0, s);
        if (!need_mask) {
#pragma unroll
          for (int i = 0; i < 32; ++i) mx = fmaxf(mx, s[i]);
        } else {
#pragma unroll
          for (int i = 0; i < 32; ++i) {
            const int key = kb * kTile + c0 + i;
            if (key <= q_pos && key < n_keys) mx = fmaxf(mx, s[i]);
          }
        }
      }
      const float m_new = fmaxf(m_run, mx * scale);
      corr = (m_run == -INFINITY) ? 0.f : fast_exp2(m_run - m_new);  // (m_new == -inf: nothing seen yet, l and o are 0 anyway)
      const float neg_m = m_new == -INFINITY ? 0.f : -m_new;       // (then every key of the block is masked)
      // pass 2: probabilities -> P (bf16, A-operand layout), row sum
      float lsum = 0.f;
#pragma unroll 1
      for (int c0 = 0; c0 < kTile; c0 += 32) {
        float s[32];
        tmem_ld32(t_addr + c0, s);
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float p[8];
          if (!need_mask) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              p[i] = fast_exp2(fmaf(s[g * 8 + i], scale, neg_m));
              lsum += p[i];
            }
          } else {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const int key = kb * kTile + c0 + g * 8 + i;
              const bool valid = key <= q_pos && key < n_keys;
              p[i] = valid ? fast_exp2(fmaf(s[g * 8 + i], scale, neg_m)) : 0.f;
              lsum += p[i];
            }
          }
          const int keyc = c0 + g * 8;  // first key of this 16-byte chunk inside the block
          const int cx = (keyc & 63) >> 3;
          *reinterpret_cast<uint4*>(sp + (keyc >> 6) * kSub + tid * 128 + ((cx ^ (tid & 7)) << 4)) = pack8(p);
        }
      }
      l_run = l_run * corr + lsum;
      m_run = m_new;
      tc_fence_before();
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    __syncthreads();
    // ---- O_blk = P V ----------------------------------------------------------------------------------------------------------
    if (tid == 128) {
      tc_fence_after();
      if (!s_abort) {
#pragma unroll
        for (int j = 0; j < 2; ++j) {
          // A = P, K-major: 16 keys further = 32 bytes = +2 in the address field.  B = V as the pages hold it, [key][dim]:
          // the dimension (N) is the contiguous one ("MN-major"), 64 of it per 128-byte row, the second 64 one sub-tile
          // (leading byte offset) further, 8 keys per 1024-byte swizzle group (stride byte offset), 16 keys = 2048 bytes.
          const uint64_t adesc = make_smem_desc(smem_u32(sp + j * kSub));
#pragma unroll
          for (int k = 0; k < 4; ++k)
            umma_bf16(tmem_base + kTile, adesc + 2 * k, make_smem_desc_mn(smem_u32(sv + (j * 4 + k) * 2048), kSub, 1024), idesc_pv,
                      (j > 0 || k > 0) ? 1u : 0u);
        }
      }
      umma_commit(&obar);
      // the next block's K loads and MMAs reuse sk / sp / TMEM: wait here until this block's MMAs have retired
      if (!mbar_wait(&obar, par, &s_abort)) s_abort = 1;
    }
    if (tid < kTile) {
      if (!mbar_wait(&obar, par, &s_abort)) s_abort = 1;
      tc_fence_after();
      const uint32_t t_addr = tmem_base + ((uint32_t)(warp * 32) << 16) + kTile;
#pragma unroll
      for (int c0 = 0; c0 < kD; c0 += 32) {
        float blk[32];
        tmem_ld32(t_addr + c0, blk);
#pragma unroll
        for (int i = 0; i < 32; ++i) o_reg[c0 + i] = fmaf(o_reg[c0 + i], corr, blk[i]);
      }
      tc_fence_before();
    }
    __syncthreads();  // sv / sp / TMEM free for the next block; s_abort settled
    if (s_abort) {
      ok = false;
      // a wait expired: before the CTA leaves (and its shared memory goes to another CTA) give this block's copies,
      // which may still be in flight, one more bounded wait to land
      if (tid == 128) {
        int none = 0;
        mbar_wait(&kbar, par, &none);
      }
      break;
    }
  }

  // ---- write ------------------------------------------------------------------------------------------------------------------
  if (tid < kTile && tid < rows) {
    const float inv = (ok && l_run > 0.f) ? 1.f / l_run : 0.f;
    uint4* dst = reinterpret_cast<uint4*>(a.out + (size_t)(row0 + tid) * a.ld_out + (size_t)h * kD);
#pragma unroll
    for (int c = 0; c < 16; ++c) {
      float f[8];
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] = o_reg[c * 8 + i] * inv;
      dst[c] = pack8(f);
    }
  }
  if (!ok && tid == 0 && a.status) atomicOr(a.status, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 4) tmem_dealloc(tmem_base, 256);
}

}  // namespace
}  // namespace mlora

using namespace mlora;

extern "C" int mlora_prefill_attention(const void* d_qkv, int64_t ld, const void* d_k_pages, const void* d_v_pages,
                                       int32_t n_pages_total, const int32_t* d_block_table, int32_t max_pages,
                                       const int32_t* d_tiles, int32_t n_tiles, int32_t Hq, int32_t Hkv, int32_t D,
                                       int32_t page_size, int32_t T, void* d_out, int64_t ld_out, int32_t* d_status,
                                       void* stream) {
  MLORA_REQUIRE(D == kD && page_size == kPS, "prefill_attention: head_dim 128 and page size 16 only (got %d, %d)", D, page_size);
  MLORA_REQUIRE(n_tiles >= 0 && T >= 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && n_pages_total > 0 && max_pages > 0,
                "prefill_attention: bad sizes");
  MLORA_REQUIRE(d_qkv && d_k_pages && d_v_pages && d_block_table && d_tiles && d_out, "prefill_attention: null pointer");
  MLORA_REQUIRE(aligned16(d_qkv) && aligned16(d_k_pages) && aligned16(d_v_pages) && aligned16(d_out) && (ld * 2) % 16 == 0 &&
                    (ld_out * 2) % 16 == 0,
                "prefill_attention: 16-byte alignment of tensors and row pitches");
  MLORA_REQUIRE(n_tiles <= 2147483647 / 4 && Hq <= 65535, "prefill_attention: too many tiles / heads");
  if (n_tiles == 0 || T == 0) return MLORA_OK;
  CUtensorMap mq, mk, mv;
  int rc = make_map(&mq, d_qkv, T, Hq * kD, ld, kTile, 64);  // only the q part of every row is mapped
  if (rc) return rc;
  rc = make_map(&mk, d_k_pages, (long long)n_pages_total * Hkv * kPS, kD, kD, kPS, 64);
  if (rc) return rc;
  rc = make_map(&mv, d_v_pages, (long long)n_pages_total * Hkv * kPS, kD, kD, kPS, 64);
  if (rc) return rc;
  constexpr int smem = 6 * kSub + 1024;  // Q, K (= P), V^T
  static std::atomic<unsigned long long> attr_done{0};
  int dev = 0;
  cudaGetDevice(&dev);
  if (!((attr_done.load(std::memory_order_acquire) >> (dev & 63)) & 1ull)) {
    cudaError_t e = cudaFuncSetAttribute(prefill_attn_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return fail(MLORA_ECUDA, "prefill_attention: cudaFuncSetAttribute: %s", cudaGetErrorString(e));
    attr_done.fetch_or(1ull << (dev & 63), std::memory_order_release);
  }
  PfArgs a{d_block_table, max_pages, d_tiles, Hq, Hkv, (bf16*)d_out, ld_out, d_status};
  prefill_attn_tc_kernel<<<dim3(n_tiles, Hq), kPfThreads, smem, (cudaStream_t)stream>>>(mq, mk, mv, a);
  count_launch();
  MLORA_CHECK_LAUNCH("prefill_attn_tc_kernel");
  return MLORA_OK;
}
