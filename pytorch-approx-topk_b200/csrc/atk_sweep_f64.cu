// Column-sweep instantiations for double inputs.
#include "atk_sweep_launch.cuh"

namespace atk {
int launch_sweep_f64(const SweepLaunch& a) { return sweep_detail::launch_sweep<double>(a); }
}  // namespace atk
