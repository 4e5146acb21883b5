#include "v1g_rollout_common.cuh"
extern "C" int v1g_rollout_bwd(V1GHandle* h, const V1GLossSpec*, const float*, const float*,
                               float*, float*, float*, float*, void*) {
  return v1g_fail(h, V1G_ESTATE, "backward rollout: work in progress");
}
