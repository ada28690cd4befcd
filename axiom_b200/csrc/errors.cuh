// errors.cuh — lets the kernel translation units leave a message where
// axb_last_error() will find it.
#pragma once

namespace axb {

// printf-style; returns `status` so call sites can `return set_error(...)`.
int set_error(int status, const char *fmt, ...);

}  // namespace axb
