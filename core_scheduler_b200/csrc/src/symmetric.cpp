// Symmetric memory context and peer-memory collectives (host side). See cs/symmetric.h.
#include "cs/symmetric.h"

namespace cs::communication {
SymmetricContext::~SymmetricContext() = default;
SymmetricBlock SymmetricContext::allocate(int64_t) { return {}; }
void SymmetricContext::release(const SymmetricBlock &) {}
at::Tensor SymmetricContext::tensor(const SymmetricBlock &, at::IntArrayRef, at::ScalarType) const { return {}; }
bool SymmetricContext::locate(const void *, int64_t, int64_t *) const { return false; }
std::shared_ptr<SymmetricContext> create_symmetric_context(const Comm &, int64_t) { return nullptr; }
bool symmetric_all_reduce(SymmetricContext &, const std::vector<at::Tensor> &, Operation) { return false; }
bool symmetric_all_gather(SymmetricContext &, const std::vector<std::vector<at::Tensor>> &, const std::vector<at::Tensor> &) { return false; }
bool symmetric_reduce_scatter(SymmetricContext &, const std::vector<at::Tensor> &, const std::vector<std::vector<at::Tensor>> &, Operation) { return false; }
bool symmetric_all_to_all(SymmetricContext &, const std::vector<at::Tensor> &, const std::vector<at::Tensor> &) { return false; }
void check_device_status(SymmetricContext &, const char *) {}
}  // namespace cs::communication
