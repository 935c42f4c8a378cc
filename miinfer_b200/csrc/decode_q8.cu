// placeholder until the streaming int8 kernel lands
#include "decode_common.cuh"
namespace b200kv {
uint32_t pick_splits_q8(const b200kv_view&, uint32_t, uint32_t, uint32_t) { return 0; }
int launch_decode_q8(const DecodeParams&, const b200kv_view&, uint32_t, cudaStream_t) { return B200KV_ERR_UNSUPPORTED; }
}
