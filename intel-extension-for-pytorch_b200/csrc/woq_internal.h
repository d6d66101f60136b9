// Small helpers shared by the translation units that implement the C ABI.
#pragma once

namespace woq {

// Records a message for woq_b200_last_error() of the calling thread and returns `code`.
int set_error(int code, const char* fmt, ...);

}  // namespace woq
