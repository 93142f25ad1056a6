#include "xkv_internal.h"
namespace xkv {
bool recon_tc_supported(const xkv_decode_params&) { return false; }
bool recon_tc_plan(const xkv_decode_params&, ReconTcPlan*) { return false; }
int recon_tc_decode(const xkv_decode_params&, const ReconTcPlan&, void*, cudaStream_t) { return XKV_ERR_UNSUPPORTED; }
}
