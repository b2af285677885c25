#include "chr_gpu.h"

#ifndef CHR_BUILD_TAG
#define CHR_BUILD_TAG "dev"
#endif

extern "C" const char *chr_nf4_version(void) { return "chr_nf4 sm_100a " CHR_BUILD_TAG; }

#include <cstdlib>

#include "nf4_common.cuh"

namespace chr {
namespace {
bool &pdl_flag() {
  static bool on = [] {
    const char *v = std::getenv("CHR_NF4_PDL");
    return !(v != nullptr && v[0] == '0');
  }();
  return on;
}
}  // namespace
bool pdl_enabled() { return pdl_flag(); }
void set_pdl_enabled(bool on) { pdl_flag() = on; }

// Poll budget of the waits for a peer GPU's flag (fused GEMV exchange, split pick).
unsigned int &peer_polls() {
  static unsigned int v = kPeerPollsDefault;
  return v;
}
}  // namespace chr

extern "C" void chr_nf4_set_peer_polls(uint32_t polls) {
  chr::peer_polls() = polls == 0 ? chr::kPeerPollsDefault : polls;
}

extern "C" void chr_nf4_set_pdl(int32_t on) { chr::set_pdl_enabled(on != 0); }
