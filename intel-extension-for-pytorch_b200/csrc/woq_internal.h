// Small helpers shared by the translation units that implement the C ABI.
#pragma once

struct woq_b200_ctx;

namespace woq {

// Records a message for woq_b200_last_error() of the calling thread and returns `code`.
int set_error(int code, const char* fmt, ...);

// CUDA device a context's buffers live on, or -1 if `ctx` is not a live context.
int ctx_device(const struct ::woq_b200_ctx* ctx);

}  // namespace woq
