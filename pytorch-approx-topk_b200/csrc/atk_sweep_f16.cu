// Column-sweep instantiations for __half inputs.
#include "atk_sweep_launch.cuh"

namespace atk {
int launch_sweep_f16(const SweepLaunch& a) { return sweep_detail::launch_sweep<__half>(a); }
}  // namespace atk
