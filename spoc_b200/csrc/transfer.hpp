// transfer.hpp — staged copies between pageable host memory and the device (transfer.cc).
#pragma once
#include <cstddef>

namespace sb200 {

// Copies at least this large, from or to pageable host memory, take the staged path.
constexpr size_t kStagedCopyMinBytes = size_t(16) << 20;

bool staged_copy_enabled();                     // SAREK_B200_STAGED_COPY=0 switches the staged path off
bool host_memory_is_pageable(const void* p);    // false for pinned / registered / managed memory
// Both return 0 or a cudaError_t value and are synchronous for the host.  after_device_work: wait first for all work
// launched on the device before the call (the ordering of a default-stream copy); a caller that orders the copy
// itself, with events, passes false so that kernels in flight keep running beside the copy.
int staged_copy_to_device(int dev, void* dst, const void* src, size_t bytes, bool after_device_work = true);
int staged_copy_to_host(int dev, void* dst, const void* src, size_t bytes, bool after_device_work = true);

}  // namespace sb200
