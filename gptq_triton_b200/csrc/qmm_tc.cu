#include "qmm_tc.cuh"

namespace gptq {

bool tc_shape_ok(int, int, int, int) { return false; }
size_t tc_ws_bytes(int, int) { return 0; }
int tc_launch(const TcArgs &, int, void *, size_t, cudaStream_t) { return GPTQ_ERR_UNSUPPORTED; }

}   // namespace gptq
