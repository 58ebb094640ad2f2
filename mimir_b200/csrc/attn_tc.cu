// placeholder until the tensor-core attention kernel lands
#include "common.cuh"
namespace mimk {
int attn_tc_supported(const mimk_attn_desc&) { return 0; }
int attn_tc(const mimk_attn_desc&, cudaStream_t) { return MIMK_E_UNSUPPORTED; }
}  // namespace mimk
