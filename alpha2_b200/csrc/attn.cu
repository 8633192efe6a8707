// Entry points of the fused attention (Backend.flashAttention / flashAttentionBackward,
// packages/core/src/interfaces.ts:127-135): pick the kernel family for the storage type.
// bf16 with head dim 64 runs on the tensor cores (attn_tc.cu); everything else — fp32
// storage (the parity mode) and other head sizes — runs the fp32 FMA kernels (attn_f32.cu).
#include "common.cuh"

namespace alpha {
int attn_f32_fwd(alpha_buf q, alpha_buf k, alpha_buf v, alpha_buf o, alpha_buf lse, const alpha_attn_params_t *p);
int attn_f32_bwd(alpha_buf q, alpha_buf k, alpha_buf v, alpha_buf o, alpha_buf d_o, alpha_buf lse, alpha_buf dq,
                 alpha_buf dk, alpha_buf dv, const alpha_attn_params_t *p);
bool attn_tc_supported(const alpha_attn_params_t *p, alpha_buf q, alpha_buf k, alpha_buf v);
int attn_tc_fwd(alpha_buf q, alpha_buf k, alpha_buf v, alpha_buf o, alpha_buf lse, const alpha_attn_params_t *p);
int attn_tc_bwd(alpha_buf q, alpha_buf k, alpha_buf v, alpha_buf o, alpha_buf d_o, alpha_buf lse, alpha_buf dq,
                alpha_buf dk, alpha_buf dv, const alpha_attn_params_t *p, alpha_buf delta_in);
}  // namespace alpha

using namespace alpha;

extern "C" {

int alpha_flash_attn_fwd(alpha_buf q, alpha_buf k, alpha_buf v, alpha_buf o, alpha_buf lse,
                         const alpha_attn_params_t *p) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(p != nullptr, "alpha_flash_attn_fwd: null params");
  if (attn_tc_supported(p, q, k, v) && (o & 15) == 0) return attn_tc_fwd(q, k, v, o, lse, p);
  return attn_f32_fwd(q, k, v, o, lse, p);
}

int alpha_flash_attn_bwd(alpha_buf q, alpha_buf k, alpha_buf v, alpha_buf o, alpha_buf d_o, alpha_buf lse, alpha_buf dq,
                         alpha_buf dk, alpha_buf dv, const alpha_attn_params_t *p) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(p != nullptr, "alpha_flash_attn_bwd: null params");
  if (attn_tc_supported(p, q, k, v) && ((o | d_o | dq | dk | dv) & 15) == 0)
    return attn_tc_bwd(q, k, v, o, d_o, lse, dq, dk, dv, p, 0);
  return attn_f32_bwd(q, k, v, o, d_o, lse, dq, dk, dv, p);
}

// The backward with the row-dots dO.O supplied by the caller (f32 [batch, heads, T], as
// alpha_gemm_nn_rowdot leaves them) instead of the forward output: tensor-core path only.
int alpha_flash_attn_bwd_delta(alpha_buf q, alpha_buf k, alpha_buf v, alpha_buf d_o, alpha_buf lse, alpha_buf delta,
                               alpha_buf dq, alpha_buf dk, alpha_buf dv, const alpha_attn_params_t *p) {
  ALPHA_REQUIRE_INIT();
  ALPHA_CHECK(p != nullptr && delta != 0, "alpha_flash_attn_bwd_delta: null argument");
  ALPHA_CHECK(attn_tc_supported(p, q, k, v) && ((d_o | dq | dk | dv) & 15) == 0,
              "alpha_flash_attn_bwd_delta: bf16, head dim 64 and 16-byte aligned tensors only; use alpha_flash_attn_bwd");
  return attn_tc_bwd(q, k, v, 0, d_o, lse, dq, dk, dv, p, delta);
}

}  // extern "C"
