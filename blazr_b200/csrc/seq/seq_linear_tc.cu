// seq_linear_tc.cu -- tensor-core path of the dense linear layer (placeholder entry points until the tcgen05 kernel is in).
#include "seq_common.cuh"

namespace b200seq {

bool linear_tc_usable(int, int64_t, int, int, int, const void*, const void*) { return false; }
int launch_linear_tc(const void*, int64_t, const void*, int, int, int, float*, int64_t, cudaStream_t) {
    return fail(B200SEQ_ERR_UNSUPPORTED, "linear: tensor-core path not built");
}

}  // namespace b200seq
