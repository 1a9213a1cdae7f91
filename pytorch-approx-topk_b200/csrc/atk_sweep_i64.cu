// Column-sweep instantiations for int64 inputs.
#include "atk_sweep_launch.cuh"

namespace atk {
int launch_sweep_i64(const SweepLaunch& a) { return sweep_detail::launch_sweep<long long>(a); }
}  // namespace atk
