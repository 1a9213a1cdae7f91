// Column-sweep instantiations for uint8 inputs.
#include "atk_sweep_launch.cuh"

namespace atk {
int launch_sweep_u8(const SweepLaunch& a) { return sweep_detail::launch_sweep<uint8_t>(a); }
}  // namespace atk
