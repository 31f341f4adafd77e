// C entry points of causal attention: validate, then route to the tcgen05 kernels (bf16, d_head 64, seq % 128 == 0)
// or to the exact-fp32 CUDA-core kernels (everything else).
#include "attn_common.cuh"

using namespace ptj;

namespace {
bool shape_ok(const ptj_attn_shape* s) {
  return s && s->batch >= 1 && s->heads >= 1 && s->seq >= 1 && s->d_head >= 1 &&
         s->batch * s->heads * s->seq < (1LL << 40);
}
AttnDropout make_dropout(float p, int train, uint64_t seed, uint32_t stream_id) {
  AttnDropout d;
  d.thr16 = dropout_threshold16(p);
  d.eval_scale = 1.f - p;
  d.train = train;
  d.seed = seed;
  d.stream_id = stream_id;
  return d;
}
}  // namespace

extern "C" size_t ptj_attn_keep_bits_bytes(const ptj_attn_shape* shape, int dtype) {
  const void* none[1] = {nullptr};
  if (!shape_ok(shape) || dtype != PTJ_BF16 || !attn_tc_supported(*shape, none, 0)) return 0;
  return attn_keep_bits_bytes(*shape);
}

extern "C" int ptj_attn_keep_bits(uint32_t* bits, const ptj_attn_shape* shape, float p, uint64_t seed, uint32_t stream_id,
                                  int dtype, void* stream) {
  if (!shape_ok(shape) || !bits || !(p >= 0.f && p <= 1.f)) return PTJ_ERR_BAD_SHAPE;
  if (ptj_attn_keep_bits_bytes(shape, dtype) == 0) return PTJ_ERR_UNSUPPORTED;
  if (!aligned16(bits)) return PTJ_ERR_MISALIGNED;
  return attn_keep_bits_tc(bits, *shape, make_dropout(p, 1, seed, stream_id), static_cast<cudaStream_t>(stream));
}

extern "C" int ptj_attn_fwd(const void* q, const void* k, const void* v, void* o, float* row_max, float* row_sum,
                            const ptj_attn_shape* shape, float p, int train, uint64_t seed, uint32_t stream_id,
                            const uint32_t* keep_bits, const int32_t* row_kstart, int dtype, void* stream) {
  if (!shape_ok(shape) || !q || !k || !v || !o || !row_max || !row_sum || !(p >= 0.f && p <= 1.f))
    return PTJ_ERR_BAD_SHAPE;
  if (dtype != PTJ_F32 && dtype != PTJ_BF16) return PTJ_ERR_DTYPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const AttnDropout dr = make_dropout(p, train, seed, stream_id);
  const void* ptrs[4] = {q, k, v, o};
  if (dtype == PTJ_BF16 && attn_tc_supported(*shape, ptrs, 4))
    return attn_fwd_tc(q, k, v, o, row_max, row_sum, keep_bits, row_kstart, *shape, dr, st);
  return attn_fwd_simt(q, k, v, o, row_max, row_sum, row_kstart, *shape, dr, dtype, st);
}

static bool bwd_uses_tc(const ptj_attn_shape* shape, int dtype) {
  const void* none[1] = {nullptr};
  return dtype == PTJ_BF16 && attn_tc_supported(*shape, none, 0);
}

extern "C" size_t ptj_attn_bwd_workspace_bytes(const ptj_attn_shape* shape, int dtype) {
  if (!shape_ok(shape) || !bwd_uses_tc(shape, dtype)) return 0;
  return attn_bwd_tc_workspace_bytes(*shape);
}

extern "C" int ptj_attn_bwd(const void* d_o, const void* q, const void* k, const void* v, const void* o,
                            const float* row_max, const float* row_sum, void* dq, void* dk, void* dv,
                            const ptj_attn_shape* shape, const ptj_attn_shape* dshape, float p, int train,
                            uint64_t seed, uint32_t stream_id, const uint32_t* keep_bits, const int32_t* row_kstart,
                            void* workspace, size_t workspace_bytes, int dtype, void* stream) {
  if (!shape_ok(shape) || !shape_ok(dshape) || !d_o || !q || !k || !v || !o || !row_max || !row_sum || !dq || !dk ||
      !dv || !(p >= 0.f && p <= 1.f))
    return PTJ_ERR_BAD_SHAPE;
  if (dshape->batch != shape->batch || dshape->heads != shape->heads || dshape->seq != shape->seq ||
      dshape->d_head != shape->d_head)
    return PTJ_ERR_BAD_SHAPE;
  if (dtype != PTJ_F32 && dtype != PTJ_BF16) return PTJ_ERR_DTYPE;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const AttnDropout dr = make_dropout(p, train, seed, stream_id);
  const void* ptrs[8] = {d_o, q, k, v, o, dq, dk, dv};
  if (dtype == PTJ_BF16 && attn_tc_supported(*shape, ptrs, 8) && attn_tc_supported(*dshape, ptrs, 0))
    return attn_bwd_tc(d_o, q, k, v, o, row_max, row_sum, dq, dk, dv, *shape, *dshape, dr, keep_bits, row_kstart,
                       workspace, workspace_bytes, st);
  return attn_bwd_simt(d_o, q, k, v, o, row_max, row_sum, dq, dk, dv, row_kstart, *shape, *dshape, dr, dtype, st);
}
