// Tensor-core varlen attention entry (tcgen05).  Declines every shape until the
// tcgen05 kernel is enabled; the caller then uses the general kernel.
#include "common.cuh"

namespace acache {
struct AttnArgs;
int attention_tc_dispatch(const AttnArgs&, int, int) { return ACACHE_EUNSUPPORTED; }
}  // namespace acache
