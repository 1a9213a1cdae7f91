// Column-sweep instantiations for int16 inputs.
#include "atk_sweep_launch.cuh"

namespace atk {
int launch_sweep_i16(const SweepLaunch& a) { return sweep_detail::launch_sweep<int16_t>(a); }
}  // namespace atk
