// Thread-local status text shared by the operator-level and model-level ABIs.
#include "common.cuh"

namespace evob {
namespace {
thread_local std::string g_error;
}

void set_error(const int code, const std::string &message) {
  const char *name = "internal";
  switch (code) {
    case kOk: name = "ok"; break;
    case kInvalidArgument: name = "invalid_argument"; break;
    case kIo: name = "io"; break;
    case kModelFormat: name = "model_format"; break;
    case kUnsupported: name = "unsupported"; break;
    case kCuda: name = "cuda"; break;
    default: break;
  }
  g_error = std::string(name) + ": " + message;
}

const char *last_error() { return g_error.c_str(); }

int fail(const int code, const std::string &message) {
  set_error(code, message);
  return code;
}

int check_launch(const char *what) {
  const cudaError_t error = cudaPeekAtLastError();
  if (error == cudaSuccess) return kOk;
  return fail(kCuda, std::string(what) + ": " + cudaGetErrorString(error));
}

}  // namespace evob
