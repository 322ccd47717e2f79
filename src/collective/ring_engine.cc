#include "collective/ring_engine.h"

#include <stdexcept>

namespace b200ccl {

struct RingEngine::State {};

RingEngine::RingEngine(const RingEngineConfig&, mem::SymmetricAllocator&, mem::SymmetricRegion&, Bootstrap*) {
    throw std::runtime_error("ring engine: not available in this build");
}
RingEngine::~RingEngine() = default;
void RingEngine::launch(Collective, const CollectiveArgs&) {}
int RingEngine::channels() const { return 0; }
int RingEngine::block_threads() const { return 0; }
std::string RingEngine::async_error() const { return ""; }

}  // namespace b200ccl
