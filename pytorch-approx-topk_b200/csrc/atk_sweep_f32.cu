// Column-sweep instantiations for float inputs.
#include "atk_sweep_launch.cuh"

namespace atk {
int launch_sweep_f32(const SweepLaunch& a) { return sweep_detail::launch_sweep<float>(a); }
}  // namespace atk
