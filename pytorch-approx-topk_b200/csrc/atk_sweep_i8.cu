// Column-sweep instantiations for int8 inputs.
#include "atk_sweep_launch.cuh"

namespace atk {
int launch_sweep_i8(const SweepLaunch& a) { return sweep_detail::launch_sweep<int8_t>(a); }
}  // namespace atk
