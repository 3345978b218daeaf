// Definition of the opaque chb_program handle shared by the C ABI sources.
#pragma once
#include "../sched/program.h"

struct chb_program {
  chb::Program prog;
};
