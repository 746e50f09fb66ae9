// Internal helpers shared by the translation units of the library.
#pragma once
#include "retarget_b200.h"

namespace rt {
int last_cuda_error_get();
void last_cuda_error_set(int e);
}  // namespace rt
