// Column-sweep instantiations for int32 inputs.
#include "atk_sweep_launch.cuh"

namespace atk {
int launch_sweep_i32(const SweepLaunch& a) { return sweep_detail::launch_sweep<int32_t>(a); }
}  // namespace atk
