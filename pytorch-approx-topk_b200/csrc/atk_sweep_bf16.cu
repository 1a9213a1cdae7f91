// Column-sweep instantiations for __nv_bfloat16 inputs.
#include "atk_sweep_launch.cuh"

namespace atk {
int launch_sweep_bf16(const SweepLaunch& a) { return sweep_detail::launch_sweep<__nv_bfloat16>(a); }
}  // namespace atk
