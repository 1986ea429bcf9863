// Greedy decode with a per-layer KV cache (placeholder until the cache kernels land).
#include "common.cuh"

extern "C" int tlnn_decode_begin(tlnn_ctx*, const tlnn_gpt_model*, const void*, int, int, int, int, int32_t*, tlnn_decoder**) {
    tl_set_error("decode is not built yet");
    return TLNN_ERR_VALUE;
}
extern "C" int tlnn_decode_step(tlnn_decoder*, const int32_t*, int32_t*) { tl_set_error("decode is not built yet"); return TLNN_ERR_VALUE; }
extern "C" int tlnn_decode_run(tlnn_decoder*, const int32_t*, int, int32_t*) { tl_set_error("decode is not built yet"); return TLNN_ERR_VALUE; }
extern "C" int tlnn_decode_end(tlnn_decoder*) { return TLNN_OK; }
