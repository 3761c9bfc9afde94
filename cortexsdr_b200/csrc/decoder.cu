// placeholder until the decoder driver lands
#include "internal.hpp"
using namespace csdr;
extern "C" {
int csdr_decoder_create(csdr_archive*, const csdr_decoder_config*, csdr_decoder**) { set_last_error("decoder not built yet"); return CSDR_ERR_UNSUPPORTED; }
int csdr_decoder_destroy(csdr_decoder*) { return CSDR_OK; }
int csdr_decoder_reset(csdr_decoder*) { return CSDR_ERR_UNSUPPORTED; }
int csdr_decoder_forward(csdr_decoder*, uint32_t, const int32_t*, size_t, float*, float*) { return CSDR_ERR_UNSUPPORTED; }
int csdr_decoder_step(csdr_decoder*, const int32_t*, size_t, int32_t*, float*) { return CSDR_ERR_UNSUPPORTED; }
int csdr_decoder_step_device_async(csdr_decoder*, const int32_t*, size_t, int32_t*) { return CSDR_ERR_UNSUPPORTED; }
int csdr_nccl_unique_id(void*) { return CSDR_ERR_UNSUPPORTED; }
int csdr_nccl_comm_create(csdr_context*, const void*, int, int, void**) { return CSDR_ERR_UNSUPPORTED; }
int csdr_nccl_comm_destroy(void*) { return CSDR_ERR_UNSUPPORTED; }
}
