// placeholder
#include "kernels.h"
namespace mlb {
bool qr_blocked_fits(uint32_t, uint32_t) { return false; }
void launch_qr_blocked(DeviceContext&, cudaStream_t, const QrProblem&) { throw std::runtime_error("qr_blocked: not built"); }
}
