// hb_query and the entry points whose kernels live in other translation units.
#include "host_common.h"

namespace hb {
int fa_smem_bytes();
int gemm_smem_bytes();
}  // namespace hb

extern "C" {

int hb_query(int what) {
  hb::clear_error();
  if (what == HB_QUERY_FA_SMEM) return hb::fa_smem_bytes();
  if (what == HB_QUERY_GEMM_SMEM) return hb::gemm_smem_bytes();
  hb::DeviceState* st = nullptr;
  if (hb::get_device_state(&st) != HB_OK) return -1;
  switch (what) {
    case HB_QUERY_SM_COUNT:
      return st->sm_count;
    case HB_QUERY_SMEM_OPTIN:
      return st->smem_optin;
    case HB_QUERY_CC:
      return st->cc;
    default:
      hb::set_error(HB_ERR_BAD_ARG, "hb_query: unknown selector %d", what);
      return -1;
  }
}

}  // extern "C"
