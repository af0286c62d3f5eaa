// sky-1 decoder block, forward and backward, as one host call each over the operators above.
//
// The dataflow is the one of the reference's DecoderExecutor (crates/sky-1/src/training/model/
// decoder.rs: train_forward :332-520, train_backward :523-695), whose operator module is missing
// from the reference tree, so only the order of operations, the saved tensors and the
// accumulate-into-f32-gradient convention are taken from it:
//   (SwiGLU is fused into the gate GEMM's and the down-projection dgrad's epilogue)
//   forward   h1 = RMSNorm(x; g1); qkv = h1 Wqkv; RoPE(q, k); attn = causal FA(q, k, v);
//             o = attn Wo + x; h2 = RMSNorm(o; g2); up = h2 Wup; gate = h2 Wgate;
//             act = SiLU(gate) * up; out = act Wdown + o.        saved: qkv attn lse o up gate act
//   backward  h1 and h2 are recomputed (decoder.rs:560-567, 660-667); weight gradients are
//             accumulated into f32 buffers (beta = 1), residual gradients are fused into the
//             RMSNorm backward (residual_dy), the second FFN dgrad accumulates into the first
//             (decoder.rs:591-596).
// Residual adds and gradient accumulation ride in the GEMM epilogue (C operand, beta = 1).
// Weights are stored [in, out] (decoder.rs:166-173).  Everything runs on the caller's stream;
// nothing is allocated: the caller passes one workspace sized by *_workspace_bytes.
#include "ops.h"


namespace cdl {
namespace {

struct Dims {
  long long T, S, B, Hd, H, Hkv, D, F, QKV;
  // ragged batch (nullptr: B sequences of S tokens): sequence b is tokens cu[b] .. cu[b + 1] of the T
  const cdl_sky1_ragged* rg = nullptr;
};

int32_t read_ragged(const cdl_sky1_ragged* rg, Dims* d) {
  d->rg = rg;
  if (!rg) return CDL_OK;
  if (!rg->cu_seqlens || rg->num_seqs <= 0 || rg->max_seqlen <= 0)
    return fail(CDL_ERR_INVALID, "sky1_block: ragged batches need cu_seqlens, num_seqs > 0 and max_seqlen > 0");
  if (rg->max_seqlen > d->T)
    return fail(CDL_ERR_INVALID, "sky1_block: max_seqlen %d exceeds the %lld tokens of the buffers",
                rg->max_seqlen, d->T);
  return CDL_OK;
}

int32_t read_config(const cdl_sky1_config* c, Dims* d) {
  if (!c) return fail(CDL_ERR_INVALID, "sky1_block: config is required");
  d->B = c->batch; d->S = c->seqlen; d->T = static_cast<long long>(c->batch) * c->seqlen;
  d->Hd = c->hidden; d->H = c->heads; d->Hkv = c->kv_heads; d->D = c->head_dim; d->F = c->ffn;
  d->QKV = (d->H + 2 * d->Hkv) * d->D;
  if (d->B <= 0 || d->S <= 0 || d->Hd <= 0 || d->H <= 0 || d->Hkv <= 0 || d->F <= 0)
    return fail(CDL_ERR_INVALID, "sky1_block: all dimensions must be positive");
  if (d->D != 128) return fail(CDL_ERR_UNSUPPORTED, "sky1_block: head_dim must be 128");
  if (d->H % d->Hkv != 0) return fail(CDL_ERR_INVALID, "sky1_block: heads must be a multiple of kv_heads");
  if (d->Hd % 8 != 0 || d->F % 8 != 0 || d->Hd > 8192)
    return fail(CDL_ERR_UNSUPPORTED, "sky1_block: hidden and ffn must be multiples of 8, hidden <= 8192");
  return CDL_OK;
}

size_t align256(size_t v) { return (v + 255) / 256 * 256; }

// Carves the workspace; with base == nullptr only the total size is computed.
struct Workspace {
  uint8_t* base;
  size_t used = 0;
  explicit Workspace(void* b) : base(static_cast<uint8_t*>(b)) {}
  void* take(size_t bytes) {
    void* p = base ? base + used : nullptr;
    used += align256(bytes);
    return p;
  }
};

struct FwdBuffers { void* h; float* r_inv; };
FwdBuffers carve_fwd(Workspace& w, const Dims& d) {
  FwdBuffers b;
  b.h = w.take(d.T * d.Hd * 2);
  b.r_inv = static_cast<float*>(w.take(d.T * 4));
  return b;
}

struct BwdBuffers {
  void* h; float* r_inv; void* dact; void* dgate; void* dh; void* d_o; void* dattn; void* dqkv;
  void* attn_scratch; size_t attn_scratch_bytes; void* norm_scratch; size_t norm_scratch_bytes;
};
BwdBuffers carve_bwd(Workspace& w, const Dims& d) {
  BwdBuffers b;
  b.h = w.take(d.T * d.Hd * 2);
  b.r_inv = static_cast<float*>(w.take(d.T * 4));
  b.dact = w.take(d.T * d.F * 2);   // d_act, then d_up in place
  b.dgate = w.take(d.T * d.F * 2);
  b.dh = w.take(d.T * d.Hd * 2);    // dh2, later dh1
  b.d_o = w.take(d.T * d.Hd * 2);
  b.dattn = w.take(d.T * d.H * d.D * 2);
  b.dqkv = w.take(d.T * d.QKV * 2);
  b.attn_scratch_bytes = d.rg ? attn_bwd_packed_scratch_bytes(d.rg->num_seqs, d.rg->max_seqlen, d.H)
                              : attn_bwd_scratch_bytes(d.B, d.S, d.H);
  b.attn_scratch = w.take(b.attn_scratch_bytes);
  b.norm_scratch_bytes = rmsnorm_bwd_scratch_bytes(d.T, d.Hd);
  b.norm_scratch = w.take(b.norm_scratch_bytes);
  return b;
}

// q / k / v views of the fused qkv buffer [T, (H + 2 Hkv) D] as [B, S, heads, D].
cdl_tensor head_view(const void* qkv, const Dims& d, long long first_head, long long heads) {
  cdl_tensor t{};
  t.ptr = static_cast<uint8_t*>(const_cast<void*>(qkv)) + first_head * d.D * 2;
  t.dtype = CDL_BF16;
  t.rank = 4;
  t.shape[0] = d.B; t.shape[1] = d.S; t.shape[2] = heads; t.shape[3] = d.D;
  t.stride[0] = d.S * d.QKV; t.stride[1] = d.QKV; t.stride[2] = d.D; t.stride[3] = 1;
  return t;
}
// The same heads of the fused qkv buffer as a packed [T, heads, D] view (ragged batches).
cdl_tensor head_view_packed(const void* qkv, const Dims& d, long long first_head, long long heads) {
  cdl_tensor t{};
  t.ptr = static_cast<uint8_t*>(const_cast<void*>(qkv)) + first_head * d.D * 2;
  t.dtype = CDL_BF16;
  t.rank = 3;
  t.shape[0] = d.T; t.shape[1] = heads; t.shape[2] = d.D;
  t.stride[0] = d.QKV; t.stride[1] = d.D; t.stride[2] = 1;
  return t;
}
cdl_tensor attn_view_packed(const void* p, const Dims& d) {
  cdl_tensor t{};
  t.ptr = const_cast<void*>(p);
  t.dtype = CDL_BF16;
  t.rank = 3;
  t.shape[0] = d.T; t.shape[1] = d.H; t.shape[2] = d.D;
  t.stride[0] = d.H * d.D; t.stride[1] = d.D; t.stride[2] = 1;
  return t;
}
cdl_tensor lse_view_packed(const float* p, const Dims& d) {  // [heads, T]
  cdl_tensor t{};
  t.ptr = const_cast<float*>(p);
  t.dtype = CDL_F32;
  t.rank = 2;
  t.shape[0] = d.H; t.shape[1] = d.T;
  t.stride[0] = d.T; t.stride[1] = 1;
  return t;
}
cdl_tensor cu_view(const Dims& d) {
  cdl_tensor t{};
  t.ptr = const_cast<int32_t*>(d.rg->cu_seqlens);
  t.dtype = CDL_I32;
  t.rank = 1;
  t.shape[0] = d.rg->num_seqs + 1;
  t.stride[0] = 1;
  return t;
}
cdl_tensor attn_view(const void* p, const Dims& d) {
  cdl_tensor t{};
  t.ptr = const_cast<void*>(p);
  t.dtype = CDL_BF16;
  t.rank = 4;
  t.shape[0] = d.B; t.shape[1] = d.S; t.shape[2] = d.H; t.shape[3] = d.D;
  t.stride[0] = d.S * d.H * d.D; t.stride[1] = d.H * d.D; t.stride[2] = d.D; t.stride[3] = 1;
  return t;
}
cdl_tensor lse_view(const float* p, const Dims& d) {
  cdl_tensor t{};
  t.ptr = const_cast<float*>(p);
  t.dtype = CDL_F32;
  t.rank = 3;
  t.shape[0] = d.B; t.shape[1] = d.H; t.shape[2] = d.S;
  t.stride[0] = d.H * d.S; t.stride[1] = d.S; t.stride[2] = 1;
  return t;
}

}  // namespace

size_t sky1_block_fwd_workspace(const Dims& d) {
  Workspace w(nullptr);
  carve_fwd(w, d);
  return w.used;
}
size_t sky1_block_bwd_workspace(const Dims& d) {
  Workspace w(nullptr);
  carve_bwd(w, d);
  return w.used;
}

int32_t sky1_block_fwd(const cdl_sky1_config* cfg, const cdl_sky1_weights* wt, const void* x,
                       const float* rope_cos_sin, const cdl_sky1_saved* sv, void* out,
                       void* workspace, size_t workspace_bytes, const cdl_sky1_ragged* rg,
                       cudaStream_t st) {
  Dims d;
  CDL_CHECK(read_config(cfg, &d));
  CDL_CHECK(read_ragged(rg, &d));
  if (!wt || !x || !rope_cos_sin || !sv || !out)
    return fail(CDL_ERR_INVALID, "sky1_block_fwd: weights, x, rope table, saved and out are required");
  if (!workspace || workspace_bytes < sky1_block_fwd_workspace(d) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(CDL_ERR_INVALID, "sky1_block_fwd: workspace must be 256-byte aligned and hold %zu bytes",
                sky1_block_fwd_workspace(d));
  Workspace w(workspace);
  const FwdBuffers b = carve_fwd(w, d);
  const long long HD = d.H * d.D;

  const cdl_tensor tx = view2(x, CDL_BF16, d.T, d.Hd), th = view2(b.h, CDL_BF16, d.T, d.Hd);
  const cdl_tensor g1 = view1(wt->norm1, CDL_BF16, d.Hd), g2 = view1(wt->norm2, CDL_BF16, d.Hd);
  const cdl_tensor tqkv = view2(sv->qkv, CDL_BF16, d.T, d.QKV);
  const cdl_tensor wqkv = view2(wt->wqkv, CDL_BF16, d.Hd, d.QKV);
  const cdl_tensor tattn = view2(sv->attn, CDL_BF16, d.T, HD), wo = view2(wt->wo, CDL_BF16, HD, d.Hd);
  const cdl_tensor to = view2(sv->o, CDL_BF16, d.T, d.Hd);
  const cdl_tensor tup = view2(sv->up, CDL_BF16, d.T, d.F), tgate = view2(sv->gate, CDL_BF16, d.T, d.F);
  const cdl_tensor tact = view2(sv->act, CDL_BF16, d.T, d.F);
  const cdl_tensor wup = view2(wt->wup, CDL_BF16, d.Hd, d.F), wgate = view2(wt->wgate, CDL_BF16, d.Hd, d.F);
  const cdl_tensor wdown = view2(wt->wdown, CDL_BF16, d.F, d.Hd);
  const cdl_tensor tout = view2(out, CDL_BF16, d.T, d.Hd);
  const long long table_rows = d.rg ? d.rg->max_seqlen : d.S;
  const cdl_attn_desc ad{0.0f, 1};

  CDL_CHECK(rmsnorm_fwd_execute(&tx, &g1, nullptr, cfg->eps, &th, nullptr, st));
  // qkv = h1 Wqkv with RoPE on the q and k heads applied in the GEMM's epilogue
  const RopeEpilogue rope{rope_cos_sin, static_cast<int>(table_rows), static_cast<int>((d.H + d.Hkv) * d.D),
                          d.rg ? d.rg->cu_seqlens : nullptr, d.rg ? d.rg->num_seqs : 0};
  CDL_CHECK(matmul_execute_epi(&th, &wqkv, nullptr, &tqkv, 1.f, 0.f, 3, nullptr, nullptr, nullptr, st, nullptr,
                               &rope));
  if (d.rg) {
    const cdl_tensor cu = cu_view(d);
    const cdl_tensor q = head_view_packed(sv->qkv, d, 0, d.H), k = head_view_packed(sv->qkv, d, d.H, d.Hkv),
                     v = head_view_packed(sv->qkv, d, d.H + d.Hkv, d.Hkv);
    const cdl_tensor ao = attn_view_packed(sv->attn, d), lse = lse_view_packed(sv->lse, d);
    // Rows after the last sequence are not written by the attention kernel; they are read by the
    // output projection and, in the backward, by dWo += attn^T d_o, so they must not hold NaNs.
    CDL_CUDA(cudaMemsetAsync(sv->attn, 0, static_cast<size_t>(d.T) * d.H * d.D * 2, st));
    CDL_CHECK(attn_fwd_packed_execute(&ad, &q, &k, &v, &cu, &cu, d.rg->max_seqlen, d.rg->max_seqlen,
                                      &ao, &lse, st));
  } else {
    const cdl_tensor q = head_view(sv->qkv, d, 0, d.H), k = head_view(sv->qkv, d, d.H, d.Hkv),
                     v = head_view(sv->qkv, d, d.H + d.Hkv, d.Hkv);
    const cdl_tensor ao = attn_view(sv->attn, d), lse = lse_view(sv->lse, d);
    CDL_CHECK(attn_fwd_execute(&ad, &q, &k, &v, &ao, &lse, st));
  }
  CDL_CHECK(matmul_execute(&tattn, &wo, &tx, &to, 1.f, 1.f, st));  // o = attn Wo + x
  CDL_CHECK(rmsnorm_fwd_execute(&to, &g2, nullptr, cfg->eps, &th, nullptr, st));
  CDL_CHECK(matmul_execute(&th, &wup, nullptr, &tup, 1.f, 0.f, st));
  // gate = h2 Wgate and act = SiLU(gate) * up in one kernel (fused epilogue)
  CDL_CHECK(matmul_execute_epi(&th, &wgate, nullptr, &tgate, 1.f, 0.f, 1, &tup, nullptr, &tact, st));
  CDL_CHECK(matmul_execute(&tact, &wdown, &to, &tout, 1.f, 1.f, st));  // out = act Wdown + o
  return CDL_OK;
}

int32_t sky1_block_bwd(const cdl_sky1_config* cfg, const cdl_sky1_weights* wt, const void* x,
                       const float* rope_cos_sin, const cdl_sky1_saved* sv, const void* dy,
                       const cdl_sky1_grads* gr, void* dx, void* workspace, size_t workspace_bytes,
                       int32_t phase, const cdl_sky1_ragged* rg, cudaStream_t st,
                       const cdl_sky1_grad_events* ev) {
  Dims d;
  CDL_CHECK(read_config(cfg, &d));
  CDL_CHECK(read_ragged(rg, &d));
  if (!wt || !x || !rope_cos_sin || !sv || !dy || !gr || !dx)
    return fail(CDL_ERR_INVALID, "sky1_block_bwd: every argument is required");
  if (!workspace || workspace_bytes < sky1_block_bwd_workspace(d) ||
      (reinterpret_cast<uintptr_t>(workspace) & 255) != 0)
    return fail(CDL_ERR_INVALID, "sky1_block_bwd: workspace must be 256-byte aligned and hold %zu bytes",
                sky1_block_bwd_workspace(d));
  Workspace w(workspace);
  const BwdBuffers b = carve_bwd(w, d);
  const long long HD = d.H * d.D;

  const cdl_tensor tx = view2(x, CDL_BF16, d.T, d.Hd), th = view2(b.h, CDL_BF16, d.T, d.Hd);
  const cdl_tensor tr = view1(b.r_inv, CDL_F32, d.T);
  const cdl_tensor g1 = view1(wt->norm1, CDL_BF16, d.Hd), g2 = view1(wt->norm2, CDL_BF16, d.Hd);
  const cdl_tensor dg1 = view1(gr->norm1, CDL_F32, d.Hd), dg2 = view1(gr->norm2, CDL_F32, d.Hd);
  const cdl_tensor tdy = view2(dy, CDL_BF16, d.T, d.Hd), tdx = view2(dx, CDL_BF16, d.T, d.Hd);
  const cdl_tensor tact = view2(sv->act, CDL_BF16, d.T, d.F), tup = view2(sv->up, CDL_BF16, d.T, d.F);
  const cdl_tensor tgate = view2(sv->gate, CDL_BF16, d.T, d.F), to = view2(sv->o, CDL_BF16, d.T, d.Hd);
  const cdl_tensor tattn = view2(sv->attn, CDL_BF16, d.T, HD);
  const cdl_tensor wqkv = view2(wt->wqkv, CDL_BF16, d.Hd, d.QKV), wo = view2(wt->wo, CDL_BF16, HD, d.Hd);
  const cdl_tensor wup = view2(wt->wup, CDL_BF16, d.Hd, d.F), wgate = view2(wt->wgate, CDL_BF16, d.Hd, d.F);
  const cdl_tensor wdown = view2(wt->wdown, CDL_BF16, d.F, d.Hd);
  const cdl_tensor gwqkv = view2(gr->wqkv, CDL_F32, d.Hd, d.QKV), gwo = view2(gr->wo, CDL_F32, HD, d.Hd);
  const cdl_tensor gwup = view2(gr->wup, CDL_F32, d.Hd, d.F), gwgate = view2(gr->wgate, CDL_F32, d.Hd, d.F);
  const cdl_tensor gwdown = view2(gr->wdown, CDL_F32, d.F, d.Hd);
  const cdl_tensor tdact = view2(b.dact, CDL_BF16, d.T, d.F), tdgate = view2(b.dgate, CDL_BF16, d.T, d.F);
  const cdl_tensor tdh = view2(b.dh, CDL_BF16, d.T, d.Hd), tdo = view2(b.d_o, CDL_BF16, d.T, d.Hd);
  const cdl_tensor tdattn = view2(b.dattn, CDL_BF16, d.T, HD), tdqkv = view2(b.dqkv, CDL_BF16, d.T, d.QKV);
  const cdl_tensor cs = view2(rope_cos_sin, CDL_F32, d.rg ? d.rg->max_seqlen : d.S, d.D);
  const cdl_attn_desc ad{0.0f, 1};
  const cdl_tensor actT = transposed(tact), hT = transposed(th), attnT = transposed(tattn);
  const cdl_tensor wdownT = transposed(wdown), wupT = transposed(wup), wgateT = transposed(wgate);
  const cdl_tensor woT = transposed(wo), wqkvT = transposed(wqkv);

  if (phase < 0 || phase > 2) return fail(CDL_ERR_INVALID, "sky1_block_bwd: phase must be 0, 1 or 2");
  // Weight-gradient products: the caller chooses between K slices that meet through f32 atomics
  // (default) and a fixed summation order.
  const cdl_matmul_options wg_opts{CDL_GEMM_AUTO, (cfg->flags & CDL_SKY1_DETERMINISTIC) ? 1 : 0};
  const cdl_matmul_options* wg = &wg_opts;
  // A data-parallel caller's events: recorded as soon as the kernels that complete a group of
  // weight gradients are enqueued, so that group's all-reduce can start while the rest runs.
  auto mark = [&](void* e) -> int32_t {
    if (ev && e) CDL_CUDA(cudaEventRecord(static_cast<cudaEvent_t>(e), st));
    return CDL_OK;
  };
  if (phase != 2) {
  // FFN
  CDL_CHECK(matmul_execute(&actT, &tdy, &gwdown, &gwdown, 1.f, 1.f, st, wg));          // dWdown += act^T dy
  CDL_CHECK(mark(ev ? ev->wdown : nullptr));
  // d_act = dy Wdown^T never reaches memory: the epilogue turns it into d_up and d_gate
  CDL_CHECK(matmul_execute_epi(&tdy, &wdownT, nullptr, &tdact, 1.f, 0.f, 2, &tgate, &tup, &tdgate, st));
  CDL_CHECK(rmsnorm_fwd_execute(&to, &g2, nullptr, cfg->eps, &th, &tr, st));        // recompute h2, r2
  CDL_CHECK(matmul_execute(&hT, &tdact, &gwup, &gwup, 1.f, 1.f, st, wg));               // dWup += h2^T d_up
  CDL_CHECK(mark(ev ? ev->wup : nullptr));
  CDL_CHECK(matmul_execute(&tdact, &wupT, nullptr, &tdh, 1.f, 0.f, st));            // dh2 = d_up Wup^T
  CDL_CHECK(matmul_execute(&hT, &tdgate, &gwgate, &gwgate, 1.f, 1.f, st, wg));          // dWgate += h2^T d_gate
  CDL_CHECK(matmul_execute(&tdgate, &wgateT, &tdh, &tdh, 1.f, 1.f, st));            // dh2 += d_gate Wgate^T
  CDL_CHECK(rmsnorm_bwd_execute(&to, &tdh, &tdy, &g2, &tr, &tdo, &dg2, b.norm_scratch,
                                b.norm_scratch_bytes, st));                         // d_o (+ dy)
  CDL_CHECK(mark(ev ? ev->wgate_norm2 : nullptr));
  }
  if (phase == 1) return CDL_OK;
  // attention
  CDL_CHECK(matmul_execute(&attnT, &tdo, &gwo, &gwo, 1.f, 1.f, st, wg));                // dWo += attn^T d_o
  CDL_CHECK(mark(ev ? ev->wo : nullptr));
  CDL_CHECK(matmul_execute(&tdo, &woT, nullptr, &tdattn, 1.f, 0.f, st));            // d_attn = d_o Wo^T
  // d_q and d_k leave the attention backward already rotated back (the transpose of the rotary
  // embedding runs in its store epilogues)
  if (d.rg) {
    const cdl_tensor cu = cu_view(d);
    // Rows after the last sequence get no gradient from the attention kernels: clear the buffer
    // so that the GEMMs that read all T rows of d_qkv see zeros there.
    CDL_CUDA(cudaMemsetAsync(b.dqkv, 0, static_cast<size_t>(d.T) * d.QKV * 2, st));
    const cdl_tensor q = head_view_packed(sv->qkv, d, 0, d.H), k = head_view_packed(sv->qkv, d, d.H, d.Hkv),
                     v = head_view_packed(sv->qkv, d, d.H + d.Hkv, d.Hkv);
    const cdl_tensor dq = head_view_packed(b.dqkv, d, 0, d.H), dk = head_view_packed(b.dqkv, d, d.H, d.Hkv),
                     dv = head_view_packed(b.dqkv, d, d.H + d.Hkv, d.Hkv);
    const cdl_tensor ao = attn_view_packed(sv->attn, d), dao = attn_view_packed(b.dattn, d),
                     lse = lse_view_packed(sv->lse, d);
    CDL_CHECK(attn_bwd_packed_execute(&ad, &q, &k, &v, &ao, &dao, &lse, &cu, &cu, d.rg->max_seqlen,
                                      d.rg->max_seqlen, &dq, &dk, &dv, b.attn_scratch,
                                      b.attn_scratch_bytes, st, &cs));
  } else {
    const cdl_tensor q = head_view(sv->qkv, d, 0, d.H), k = head_view(sv->qkv, d, d.H, d.Hkv),
                     v = head_view(sv->qkv, d, d.H + d.Hkv, d.Hkv);
    const cdl_tensor dq = head_view(b.dqkv, d, 0, d.H), dk = head_view(b.dqkv, d, d.H, d.Hkv),
                     dv = head_view(b.dqkv, d, d.H + d.Hkv, d.Hkv);
    const cdl_tensor ao = attn_view(sv->attn, d), dao = attn_view(b.dattn, d), lse = lse_view(sv->lse, d);
    CDL_CHECK(attn_bwd_execute(&ad, &q, &k, &v, &ao, &dao, &lse, &dq, &dk, &dv, b.attn_scratch,
                               b.attn_scratch_bytes, st, &cs));
  }
  CDL_CHECK(rmsnorm_fwd_execute(&tx, &g1, nullptr, cfg->eps, &th, &tr, st));        // recompute h1, r1
  CDL_CHECK(matmul_execute(&hT, &tdqkv, &gwqkv, &gwqkv, 1.f, 1.f, st, wg));             // dWqkv += h1^T d_qkv
  CDL_CHECK(matmul_execute(&tdqkv, &wqkvT, nullptr, &tdh, 1.f, 0.f, st));           // dh1 = d_qkv Wqkv^T
  CDL_CHECK(rmsnorm_bwd_execute(&tx, &tdh, &tdo, &g1, &tr, &tdx, &dg1, b.norm_scratch,
                                b.norm_scratch_bytes, st));                         // dx (+ d_o)
  CDL_CHECK(mark(ev ? ev->wqkv_norm1 : nullptr));
  return CDL_OK;
}

}  // namespace cdl

extern "C" {

int32_t cdl_b200_sky1_block_workspace_bytes_ragged(const cdl_sky1_config* cfg,
                                                   const cdl_sky1_ragged* ragged, size_t* fwd_bytes,
                                                   size_t* bwd_bytes) {
  cdl::Dims d;
  CDL_CHECK(cdl::read_config(cfg, &d));
  CDL_CHECK(cdl::read_ragged(ragged, &d));
  if (fwd_bytes) *fwd_bytes = cdl::sky1_block_fwd_workspace(d);
  if (bwd_bytes) *bwd_bytes = cdl::sky1_block_bwd_workspace(d);
  return CDL_OK;
}

int32_t cdl_b200_sky1_block_fwd_ragged(const cdl_sky1_config* cfg, const cdl_sky1_weights* weights,
                                       const void* x, const float* rope_cos_sin,
                                       const cdl_sky1_ragged* ragged, const cdl_sky1_saved* saved,
                                       void* out, void* workspace, size_t workspace_bytes,
                                       cdl_stream stream) {
  if (!ragged) return cdl::fail(CDL_ERR_INVALID, "sky1_block_fwd_ragged: the ragged descriptor is required");
  return cdl::sky1_block_fwd(cfg, weights, x, rope_cos_sin, saved, out, workspace, workspace_bytes,
                             ragged, static_cast<cudaStream_t>(stream));
}

int32_t cdl_b200_sky1_block_bwd_ragged(const cdl_sky1_config* cfg, const cdl_sky1_weights* weights,
                                       const void* x, const float* rope_cos_sin,
                                       const cdl_sky1_ragged* ragged, const cdl_sky1_saved* saved,
                                       const void* dy, const cdl_sky1_grads* grads, void* dx,
                                       void* workspace, size_t workspace_bytes, int32_t phase,
                                       cdl_stream stream) {
  if (!ragged) return cdl::fail(CDL_ERR_INVALID, "sky1_block_bwd_ragged: the ragged descriptor is required");
  return cdl::sky1_block_bwd(cfg, weights, x, rope_cos_sin, saved, dy, grads, dx, workspace,
                             workspace_bytes, phase, ragged, static_cast<cudaStream_t>(stream), nullptr);
}

int32_t cdl_b200_sky1_block_workspace_bytes(const cdl_sky1_config* cfg, size_t* fwd_bytes,
                                            size_t* bwd_bytes) {
  cdl::Dims d;
  CDL_CHECK(cdl::read_config(cfg, &d));
  if (fwd_bytes) *fwd_bytes = cdl::sky1_block_fwd_workspace(d);
  if (bwd_bytes) *bwd_bytes = cdl::sky1_block_bwd_workspace(d);
  return CDL_OK;
}

int32_t cdl_b200_sky1_block_fwd(const cdl_sky1_config* cfg, const cdl_sky1_weights* weights,
                                const void* x, const float* rope_cos_sin,
                                const cdl_sky1_saved* saved, void* out, void* workspace,
                                size_t workspace_bytes, cdl_stream stream) {
  return cdl::sky1_block_fwd(cfg, weights, x, rope_cos_sin, saved, out, workspace, workspace_bytes,
                             nullptr, static_cast<cudaStream_t>(stream));
}

int32_t cdl_b200_sky1_block_bwd(const cdl_sky1_config* cfg, const cdl_sky1_weights* weights,
                                const void* x, const float* rope_cos_sin,
                                const cdl_sky1_saved* saved, const void* dy,
                                const cdl_sky1_grads* grads, void* dx, void* workspace,
                                size_t workspace_bytes, int32_t phase, cdl_stream stream) {
  return cdl::sky1_block_bwd(cfg, weights, x, rope_cos_sin, saved, dy, grads, dx, workspace,
                             workspace_bytes, phase, nullptr, static_cast<cudaStream_t>(stream), nullptr);
}

int32_t cdl_b200_sky1_block_bwd_events(const cdl_sky1_config* cfg, const cdl_sky1_weights* weights,
                                       const void* x, const float* rope_cos_sin,
                                       const cdl_sky1_ragged* ragged, const cdl_sky1_saved* saved,
                                       const void* dy, const cdl_sky1_grads* grads, void* dx,
                                       void* workspace, size_t workspace_bytes,
                                       const cdl_sky1_grad_events* events, cdl_stream stream) {
  return cdl::sky1_block_bwd(cfg, weights, x, rope_cos_sin, saved, dy, grads, dx, workspace,
                             workspace_bytes, 0, ragged, static_cast<cudaStream_t>(stream), events);
}

}  // extern "C"
