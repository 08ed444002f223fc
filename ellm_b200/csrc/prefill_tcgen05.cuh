// K1 (fast form): causal grouped-query flash-attention prefill on tcgen05 / TMEM / TMA.
#pragma once
#include "../../include/ellm_attn.h"
#include "common.cuh"

namespace ellm {

struct Tcgen05Plan {
    bool ready = false;
    char why[160] = "not built yet";
};

inline void tcgen05_plan_init(Tcgen05Plan&, const ellm_attn_desc&, int) {}
inline bool tcgen05_prefers(const Tcgen05Plan&, size_t, int) { return false; }
inline int launch_prefill_tcgen05(Tcgen05Plan&, const ellm_attn_desc&, const int32_t*, size_t, size_t, size_t,
                                  float*, int*, cudaStream_t) {
    return ELLM_ERR_UNSUPPORTED;
}

}  // namespace ellm
