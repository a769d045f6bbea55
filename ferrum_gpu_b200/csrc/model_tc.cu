// bf16 tensor-core passes of the resident model (scoring / forward_all with FC_TENSOR_BF16).
#include "model.cuh"

int k_qgemm_tc(FcDevice* dev, FcQWeight*, const float*, uint32_t, float*) {
  return fc_fail(dev, FC_ERR_UNSUPPORTED, "the bf16 tensor-core product is not built yet");
}
int model_trunk_tc(FcModel* m, const int32_t*, const int32_t*, uint32_t, uint32_t, __nv_bfloat16*) {
  return fc_fail(m->dev, FC_ERR_UNSUPPORTED, "the bf16 tensor-core path is not built yet");
}
int model_head_partial_tc(FcModel* m, const __nv_bfloat16*, const int32_t*, uint32_t, float*) {
  return fc_fail(m->dev, FC_ERR_UNSUPPORTED, "the bf16 tensor-core path is not built yet");
}
int model_logits_tc(FcModel* m, const __nv_bfloat16*, uint32_t, float*) {
  return fc_fail(m->dev, FC_ERR_UNSUPPORTED, "the bf16 tensor-core path is not built yet");
}
void model_tc_free(FcModel*) {}
