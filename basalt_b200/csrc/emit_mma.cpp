// CTA-wide lowerings of `mma` (register-tiled FFMA for f32, TMA + tcgen05 for f16).
#include "emit.hpp"

namespace basalt {

bool emit_mma_fast(const MmaSite&, const std::string&, std::vector<std::string>*, std::vector<std::string>*, std::vector<std::string>*) {
    return false;
}

}  // namespace basalt
