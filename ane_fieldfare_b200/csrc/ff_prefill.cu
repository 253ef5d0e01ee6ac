// Prefill path: router for many rows, device-side permute, grouped INT4->bf16 tensor-core GEMMs.
#include "ff_internal.cuh"

namespace ff {

bool prefill_prepare_layer(FFContext *, LayerStore &, const char **error) {
    return fail(error, "prefill path is not built");
}
bool launch_prefill_routed(FFContext *, LayerStore &, const uint16_t *, uint32_t, uint32_t,
                           const uint32_t *, uint16_t *, cudaStream_t, const char **error) {
    return fail(error, "prefill path is not built");
}
bool launch_prefill_shared(FFContext *, LayerStore &, const uint16_t *, uint32_t, uint32_t,
                           uint16_t *, cudaStream_t, const char **error) {
    return fail(error, "prefill path is not built");
}
bool launch_router_prefill(FFContext *, const LayerStore &, const uint16_t *, uint32_t, uint32_t,
                           uint32_t *, uint16_t *, float *, cudaStream_t, const char **error) {
    return fail(error, "prefill path is not built");
}

}  // namespace ff

extern "C" bool ff_last_prefill_routes(FFContext *, FFTokenExpertPair *, uint32_t *,
                                       const char **error) {
    return ff::fail(error, "prefill path is not built");
}
