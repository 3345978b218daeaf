// Definition of the opaque chb_program handle shared by the C ABI sources.
#pragma once
#include "../sched/program.h"

#include <atomic>
#include <cstdint>

struct chb_program {
  chb::Program prog;
  // Process-unique identity: device-side copies are cached per communicator
  // under this id, never under the object's address (which can be reused).
  uint64_t uid = next_uid();
  static uint64_t next_uid() {
    static std::atomic<uint64_t> counter{1};
    return counter.fetch_add(1);
  }
};
