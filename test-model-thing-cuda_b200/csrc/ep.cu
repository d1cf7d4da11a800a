// Expert parallelism over NCCL (placeholder until the exchange path is built).
#include <stdexcept>
#include "moe_internal.h"

namespace tmt {
void ep_forward(tmt_moe*, const void*, const void*, const void* const*, const void* const*, void*, float, int) {
    throw std::runtime_error("expert parallelism is not initialised on this handle");
}
void ep_backward(tmt_moe*, const void*, const void*, const void* const*, const void* const*, float*, float* const*,
                 float* const*, void*, float, float) {
    throw std::runtime_error("expert parallelism is not initialised on this handle");
}
void ep_teardown(tmt_moe*) {}
}  // namespace tmt

extern "C" {
int tmt_moe_ep_unique_id(void*) { tmt::set_error("expert parallelism is not built yet"); return -1; }
int tmt_moe_ep_init(tmt_moe*, const void*) { tmt::set_error("expert parallelism is not built yet"); return -1; }
}
