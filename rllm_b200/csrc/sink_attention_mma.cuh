// placeholder until the tensor-core kernel lands
#pragma once
RLLM_API int rllm_sink_attention_mma_supported(int dt, int kd, int vd, int page_size) { return 0; }
RLLM_API int rllm_sink_attention_mma() { return ERR_BAD_SIZE; }
