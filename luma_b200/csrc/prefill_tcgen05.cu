// placeholder until the tcgen05 kernel lands
#include "common.cuh"
namespace fa {
int launch_prefill_tcgen05(const AttnParams&, cudaStream_t) { return -1; }
}
