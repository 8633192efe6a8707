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
                alpha_buf dk, alpha_buf dv, const alpha_attn_params_t *p);
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
    return attn_tc_bwd(q, k, v, o, d_o, lse, dq, dk, dv, p);
  return attn_f32_bwd(q, k, v, o, d_o, lse, dq, dk, dv, p);
}

}  // extern "C"
