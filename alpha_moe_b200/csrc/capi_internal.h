// Shared by the translation units of the C ABI library: the per-thread error message behind
// alpha_moe_b200_last_error().
#pragma once

namespace amoe_capi {
// Stores a printf-style message for the calling thread and returns `code`.
int fail(int code, const char* fmt, ...);
}  // namespace amoe_capi
