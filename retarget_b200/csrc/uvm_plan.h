// Plan-command grammar of the UVM control socket: one text line in, a list of
// migration requests (or the socket's error string) out.
#pragma once
#include <cstddef>
#include <cstdint>
#include <vector>

#include "retarget_b200.h"

namespace rt {

// Returns nullptr when the plan is accepted (ranges filled, possibly empty) or
// the error string the socket sends back.  `line` is not modified.
const char *expand_plan_line(const rt_alloc_info *registry, size_t n_alloc, uint64_t generation,
                             const char *line, uint64_t page, std::vector<rt_id_range> &ranges);

// Unsigned decimal with overflow check; false on any other character.
bool parse_u64(const char *word, size_t len, uint64_t *out);

}  // namespace rt
