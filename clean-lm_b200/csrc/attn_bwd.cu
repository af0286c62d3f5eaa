// placeholder until the attention backward kernel lands
#include "host.h"
extern "C" {
int32_t cdl_b200_attn_bwd(const cdl_attn_desc*, const cdl_tensor*, const cdl_tensor*,
                          const cdl_tensor*, const cdl_tensor*, const cdl_tensor*,
                          const cdl_tensor*, const cdl_tensor*, const cdl_tensor*,
                          const cdl_tensor*, void*, size_t, cdl_stream) {
  return cdl::fail(CDL_ERR_UNSUPPORTED, "attention backward is not built yet");
}
int32_t cdl_b200_attn_bwd_scratch_bytes(const cdl_tensor*, const cdl_tensor*, size_t* out) {
  if (out) *out = 0;
  return CDL_OK;
}
}
