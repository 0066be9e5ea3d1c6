// Caching allocator for page-locked host memory plus a registry of pinned
// ranges (is_pinned).
//
// Parity: torch_mlu/csrc/aten/util/memory_allocator.h:97-255 -- a best-fit set
// of free host chunks; a chunk that was the source or destination of an
// asynchronous copy is reused only after a notifier recorded on the copying
// queue has been reached; pinMemory / isPinned helpers.
#pragma once
#include <c10/core/Allocator.h>
#include "queue.h"

namespace catch_b200 {

c10::Allocator* getB200PinnedAllocator();
bool isPinnedPtr(const void* p);
// Mark that `q` reads or writes the pinned block containing `p`.
void pinnedRecordQueue(const void* p, const Queue& q);
void pinnedEmptyCache();
size_t pinnedCachedBytes();

}  // namespace catch_b200
