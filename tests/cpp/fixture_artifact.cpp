// A hand-written one-specialization artifact: a DSO that exports
// vecops_kernel_query_v1 and records what the runtime forwards to it.  The
// same role the reference gives tests/runtime/WorkspaceContextFixture.cpp:
// prove that context, stream, flags and workspace cross the C ABI untouched.
#include <cstdint>

#include "fixture_artifact.h"
#include "vecops_b200/kernel_abi.h"

namespace {

int32_t workspace(const VecopsCall* call, uint64_t* bytes, VecopsError*) {
  if (call == nullptr || bytes == nullptr || call->context == nullptr || call->context->user_data == nullptr)
    return VECOPS_STATUS_INVALID_ARGUMENT;
  auto* seen = static_cast<FixtureObservation*>(call->context->user_data);
  ++seen->workspace_queries;
  *bytes = kFixtureWorkspaceBytes;
  return VECOPS_STATUS_OK;
}

int32_t run(const VecopsCall* call, VecopsError* error) {
  if (call == nullptr || call->context == nullptr || call->context->user_data == nullptr) return VECOPS_STATUS_INVALID_ARGUMENT;
  auto* seen = static_cast<FixtureObservation*>(call->context->user_data);
  if (seen->fail_next_run) {
    if (error != nullptr && error->message != nullptr && error->message_capacity > 8) {
      const char text[] = "boom";
      for (int i = 0; i < 5; ++i) error->message[i] = text[i];
    }
    return VECOPS_STATUS_EXECUTION_ERROR;
  }
  ++seen->runs;
  seen->stream = call->context->stream;
  seen->flags = call->context->flags;
  seen->workspace = call->workspace;
  seen->workspace_size = call->workspace_size;
  seen->num_values = call->num_values;
  if (call->workspace != nullptr) static_cast<unsigned char*>(call->workspace)[0] = 0x5a;
  return VECOPS_STATUS_OK;
}

const VecopsKernelDescriptorV1 kDescriptor{
    sizeof(VecopsKernelDescriptorV1), VECOPS_KERNEL_ABI_VERSION_MAJOR, VECOPS_KERNEL_ABI_VERSION_MINOR,
    "test::fixture", "fixture-v1", 0, sizeof(VecopsParameterDescriptor), nullptr, workspace, run, 0};

}  // namespace

extern "C" VECOPS_B200_EXPORT const VecopsKernelDescriptorV1* vecops_kernel_query_v1(void) { return &kDescriptor; }
