// mlora_linear: argument checks and kernel selection for the projection path.
#include "linear.cuh"

using namespace mlora;

extern "C" size_t mlora_linear_workspace(int32_t T, int32_t in, int32_t out) {
  return linear_tc_workspace(T, in, out);
}

extern "C" int mlora_linear_plan(int32_t T, int32_t in, int32_t out, int32_t* h_plan12) {
  MLORA_REQUIRE(T > 0 && in > 0 && out > 0 && h_plan12, "linear_plan: bad arguments");
  linear_tc_plan(T, in, out, h_plan12);
  return MLORA_OK;
}

static size_t pre_offset(int32_t T, int32_t in, int32_t out) { return (linear_tc_workspace(T, in, out) + 255) & ~(size_t)255; }

extern "C" size_t mlora_linear_workspace_flags(int32_t T, int32_t in, int32_t out, int32_t flags) {
  if ((flags & MLORA_SILU_MUL) && (flags & MLORA_LORA_PER_ROW) && T > 0 && out > 0)
    return pre_offset(T, in, out) + (size_t)T * out * sizeof(float);  // + the fp32 pre-activations of the gate/up rows
  return linear_tc_workspace(T, in, out);
}

// d_A_all != NULL: the shrink is part of this call (its kernel is launched first).
static int linear_impl(const void* d_x, int64_t ldx, const void* d_W, void* d_y, int64_t ldy, int32_t T, int32_t in,
                       int32_t out, const void* d_A_all, const float* d_u, const void* d_B_all,
                       const int32_t* d_ranks, const float* d_scales, const int32_t* d_slots, int32_t n_adapters,
                       int32_t r_max, int32_t n_mod, const int32_t* h_mod_offsets, int32_t flags, void* d_work,
                       size_t work_bytes, void* stream, const NormFuse* nf = nullptr) {
  MLORA_REQUIRE(T >= 0 && in > 0 && out > 0, "linear: bad sizes T=%d in=%d out=%d", T, in, out);
  MLORA_REQUIRE(in % 8 == 0 && ldx % 8 == 0, "linear: in and ldx must be multiples of 8 (in=%d ldx=%lld)", in,
                (long long)ldx);
  MLORA_REQUIRE(d_x && d_W && d_y, "linear: null pointer");
  MLORA_REQUIRE(aligned16(d_x) && aligned16(d_W), "linear: x and W must be 16-byte aligned");
  if (flags & MLORA_SILU_MUL) MLORA_REQUIRE(out % 16 == 0, "linear: SILU_MUL needs out %% 16 == 0 (out=%d)", out);
  LinearArgs a{};
  a.x = (const bf16*)d_x;
  a.ldx = ldx;
  a.W = (const bf16*)d_W;
  a.y = d_y;
  a.ldy = ldy;
  a.T = T;
  a.in = in;
  a.out = out;
  a.flags = flags;
  a.n_mod = 1;
  a.r_max = 0;
  if (d_u) {
    MLORA_REQUIRE(d_B_all && d_ranks && d_scales && d_slots, "linear: LoRA operands missing");
    MLORA_REQUIRE(r_max > 0 && n_mod >= 1 && n_mod <= 8 && n_adapters > 0, "linear: bad r_max=%d / n_mod=%d / n_adapters=%d",
                  r_max, n_mod, n_adapters);
    MLORA_REQUIRE(aligned16(d_B_all), "linear: B_all must be 16-byte aligned");
    if (flags & MLORA_SILU_MUL) MLORA_REQUIRE(n_mod == 2, "linear: SILU_MUL implies n_mod == 2");
    MLORA_REQUIRE(r_max % 8 == 0, "linear: r_max must be a multiple of 8 (r_max=%d)", r_max);
    a.u = d_u;
    a.B_all = (const bf16*)d_B_all;
    a.ranks = d_ranks;
    a.scales = d_scales;
    a.slots = d_slots;
    a.r_max = r_max;
    a.n_mod = n_mod;
    a.n_adapters = n_adapters;
    if (flags & MLORA_SILU_MUL) {
      // interleaved gate/up: B rows are [gate half | up half] with the other module's half zero, so the
      // expand is one dot product of length 2*r_max against u = [u_gate | u_up]
      a.r_max = 2 * r_max;
      a.n_mod = 1;
      a.full_rank = 1;
      a.mod_off[0] = 0;
      a.mod_off[1] = out;
    } else if (n_mod > 1) {
      MLORA_REQUIRE(h_mod_offsets, "linear: n_mod > 1 needs module offsets");
      MLORA_REQUIRE(h_mod_offsets[0] == 0 && h_mod_offsets[n_mod] == out, "linear: module offsets must span [0,out]");
      for (int m = 0; m <= n_mod; ++m) a.mod_off[m] = h_mod_offsets[m];
    } else {
      a.mod_off[0] = 0;
      a.mod_off[1] = out;
    }
  }
  if (T == 0) return MLORA_OK;
  cudaStream_t st = (cudaStream_t)stream;
  if (nf && (nf->res || nf->sumsq_in)) {
    // residual + RMSNorm folded into the epilogues: only the decode-size instantiations of the tensor-core kernel do it
    MLORA_REQUIRE(T <= 32, "linear_norm: at most 32 rows (T=%d)", T);
    MLORA_REQUIRE(!(flags & (MLORA_FORCE_SIMT | MLORA_LORA_PER_ROW | MLORA_B_SPLIT)) && d_work && linear_tc_supported(a),
                  "linear_norm: needs the tensor-core kernel (scratch buffer, 16-byte aligned operands, no per-row expand)");
    if (nf->res) {
      MLORA_REQUIRE(nf->norm_w && nf->sumsq_out && nf->ld_res >= out, "linear_norm: residual form needs norm_w, sumsq_out, ld_res >= out");
      MLORA_REQUIRE(!(flags & (MLORA_SILU_MUL | MLORA_OUT_F32)), "linear_norm: the residual form writes bf16 rows without activation");
    }
    if (nf->sumsq_in)
      MLORA_REQUIRE(nf->n_sumsq_in > 0 && nf->norm_dim > 0 && nf->eps >= 0.f, "linear_norm: bad n_sumsq_in=%d / norm_dim=%d",
                    nf->n_sumsq_in, nf->norm_dim);
    a.nf = *nf;
    return launch_linear_tc(a, d_work, work_bytes, st);
  }
  if (d_A_all) {
    MLORA_REQUIRE(d_u && aligned16(d_A_all) && aligned16(d_u), "lora_linear: A_all and u must be non-null and 16-byte aligned");
    const int rc = mlora_lora_shrink(d_x, ldx, d_A_all, d_ranks, d_slots, n_adapters, T, in, r_max, n_mod,
                                     const_cast<float*>(d_u), stream);
    if (rc != MLORA_OK) return rc;
  }
  if ((flags & MLORA_LORA_PER_ROW) && (flags & MLORA_SILU_MUL) && d_u && lora_expand_silu_supported(a) &&
      work_bytes >= mlora_linear_workspace_flags(T, in, out, flags) && d_work) {
    // many distinct adapters in front of SiLU*up: the projection writes fp32 pre-activations of the interleaved gate / up
    // rows into the tail of the scratch buffer, the per-row expand adds each row's adapter there and applies the activation
    LinearArgs b = a;
    b.u = nullptr;
    b.B_all = nullptr;
    b.flags = (b.flags & ~(MLORA_SILU_MUL | MLORA_B_PACKED | MLORA_LORA_PER_ROW)) | MLORA_OUT_F32;
    float* pre = reinterpret_cast<float*>(static_cast<uint8_t*>(d_work) + pre_offset(T, in, out));
    b.y = pre;
    b.ldy = out;
    int rc;
    if (!(flags & MLORA_FORCE_SIMT) && linear_tc_supported(b)) {
      rc = launch_linear_tc(b, d_work, work_bytes, st);
    } else {
      MLORA_REQUIRE(!(flags & MLORA_W_PACKED), "linear: a packed weight needs the tensor-core kernel");
      rc = launch_linear_simt(b, st);
    }
    if (rc != MLORA_OK) return rc;
    LinearArgs e = a;
    e.y_in = pre;
    return launch_lora_expand_rows(e, st);
  }
  if ((flags & MLORA_LORA_PER_ROW) && d_u && lora_expand_rows_supported(a)) {
    // many distinct adapters per token tile: base projection first, then the expand laid out by (row, output feature)
    LinearArgs b = a;
    b.u = nullptr;
    b.B_all = nullptr;
    b.flags &= ~(MLORA_B_PACKED | MLORA_B_SPLIT | MLORA_LORA_PER_ROW);
    int rc;
    if (flags & MLORA_W_PACKED) {
      MLORA_REQUIRE(!(flags & MLORA_FORCE_SIMT) && d_work && linear_tc_supported(b),
                    "linear: a packed weight needs the tensor-core kernel (scratch buffer, 16-byte aligned operands)");
      rc = launch_linear_tc(b, d_work, work_bytes, st);
    } else if (!(flags & MLORA_FORCE_SIMT) && d_work && linear_tc_supported(b)) {
      rc = launch_linear_tc(b, d_work, work_bytes, st);
    } else {
      rc = launch_linear_simt(b, st);
    }
    if (rc != MLORA_OK) return rc;
    return launch_lora_expand_rows(a, st);
  }
  MLORA_REQUIRE(!(flags & MLORA_B_SPLIT), "linear: the split B layout is read by the per-row expand only "
                "(MLORA_LORA_PER_ROW, not MLORA_SILU_MUL, not MLORA_B_PACKED)");
  if (flags & MLORA_B_PACKED)
    MLORA_REQUIRE(d_u && !(flags & MLORA_FORCE_SIMT) && d_work, "linear: a packed B_all needs the tensor-core kernel");
  if (flags & (MLORA_W_PACKED | MLORA_B_PACKED)) {
    MLORA_REQUIRE(!(flags & MLORA_FORCE_SIMT) && d_work && linear_tc_supported(a),
                  "linear: a packed weight needs the tensor-core kernel (scratch buffer, 16-byte aligned operands)");
    return launch_linear_tc(a, d_work, work_bytes, st);
  }
  if (!(flags & MLORA_FORCE_SIMT) && d_work && linear_tc_supported(a))
    return launch_linear_tc(a, d_work, work_bytes, st);
  return launch_linear_simt(a, st);
}

extern "C" int mlora_linear(const void* d_x, int64_t ldx, const void* d_W, void* d_y, int64_t ldy, int32_t T,
                            int32_t in, int32_t out, const float* d_u, const void* d_B_all,
                            const int32_t* d_ranks, const float* d_scales, const int32_t* d_slots,
                            int32_t n_adapters, int32_t r_max, int32_t n_mod, const int32_t* h_mod_offsets,
                            int32_t flags, void* d_work, size_t work_bytes, void* stream) {
  return linear_impl(d_x, ldx, d_W, d_y, ldy, T, in, out, nullptr, d_u, d_B_all, d_ranks, d_scales, d_slots,
                     n_adapters, r_max, n_mod, h_mod_offsets, flags, d_work, work_bytes, stream);
}

extern "C" int mlora_linear_norm(const void* d_x, int64_t ldx, const void* d_W, void* d_y, int64_t ldy, int32_t T,
                                 int32_t in, int32_t out, const float* d_u, const void* d_B_all,
                                 const int32_t* d_ranks, const float* d_scales, const int32_t* d_slots,
                                 int32_t n_adapters, int32_t r_max, int32_t n_mod, const int32_t* h_mod_offsets,
                                 int32_t flags, void* d_work, size_t work_bytes, float* d_res, int64_t ld_res,
                                 const void* d_norm_w, float* d_sumsq_out, const float* d_sumsq_in,
                                 int32_t n_sumsq_in, float eps, int32_t norm_dim, void* stream) {
  MLORA_REQUIRE(d_res || d_sumsq_in, "linear_norm: neither a residual to update nor row sums to apply (use mlora_linear)");
  NormFuse nf{d_res, ld_res, (const bf16*)d_norm_w, d_sumsq_out, d_sumsq_in, n_sumsq_in, eps, norm_dim};
  return linear_impl(d_x, ldx, d_W, d_y, ldy, T, in, out, nullptr, d_u, d_B_all, d_ranks, d_scales, d_slots,
                     n_adapters, r_max, n_mod, h_mod_offsets, flags, d_work, work_bytes, stream, &nf);
}

extern "C" int mlora_lora_linear(const void* d_x, int64_t ldx, const void* d_W, void* d_y, int64_t ldy, int32_t T,
                                 int32_t in, int32_t out, const void* d_A_all, float* d_u, const void* d_B_all,
                                 const int32_t* d_ranks, const float* d_scales, const int32_t* d_slots,
                                 int32_t n_adapters, int32_t r_max, int32_t n_mod,
                                 const int32_t* h_mod_offsets, int32_t flags, void* d_work, size_t work_bytes,
                                 void* stream) {
  MLORA_REQUIRE(d_A_all && d_u, "lora_linear: A_all and the u scratch are required");
  return linear_impl(d_x, ldx, d_W, d_y, ldy, T, in, out, d_A_all, d_u, d_B_all, d_ranks, d_scales, d_slots,
                     n_adapters, r_max, n_mod, h_mod_offsets, flags, d_work, work_bytes, stream);
}

extern "C" size_t mlora_packed_weight_bytes(int32_t out, int32_t in) {
  if (out <= 0 || in <= 0) return 0;
  return packed_weight_bytes(out, in);
}

extern "C" int mlora_pack_weight(const void* d_W, int32_t out, int32_t in, void* d_Wp, void* stream) {
  MLORA_REQUIRE(out > 0 && in > 0 && in % 8 == 0, "pack_weight: in must be a positive multiple of 8 (out=%d in=%d)", out, in);
  MLORA_REQUIRE(d_W && d_Wp && aligned16(d_W) && aligned16(d_Wp), "pack_weight: pointers must be non-null and 16-byte aligned");
  return launch_pack_weight(d_W, out, in, d_Wp, (cudaStream_t)stream);
}

extern "C" size_t mlora_packed_lora_b_bytes(int32_t n_adapters, int32_t out, int32_t r_max) {
  if (n_adapters <= 0 || out <= 0 || r_max <= 0) return 0;
  return packed_lora_b_bytes(n_adapters, out, r_max);
}

extern "C" int mlora_pack_lora_b(const void* d_B_all, int32_t n_adapters, int32_t out, int32_t r_max, void* d_Bp,
                                 void* stream) {
  MLORA_REQUIRE(n_adapters > 0 && out > 0, "pack_lora_b: bad sizes");
  MLORA_REQUIRE(d_B_all && d_Bp && aligned16(d_B_all) && aligned16(d_Bp),
                "pack_lora_b: pointers must be non-null and 16-byte aligned");
  return launch_pack_lora_b(d_B_all, n_adapters, out, r_max, d_Bp, (cudaStream_t)stream);
}
