#include "vq_common.cuh"
namespace vq {
int launch_prefill_tensor(const VqPrefillArgs *a, cudaStream_t stream) { (void)a; (void)stream; return VQ_EUNSUPPORTED; }
}
