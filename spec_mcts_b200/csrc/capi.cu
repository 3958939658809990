// Status strings and ABI version of the q40b200 library.
#include "q40_common.cuh"

extern "C" int q40_abi_version(void) { return 1; }

extern "C" const char* q40_strerror(int status) {
  switch (status) {
    case Q40_OK: return "ok";
    case Q40_E_NULL: return "q40: a required pointer is NULL";
    case Q40_E_SHAPE: return "q40: a size violates a divisibility or range rule";
    case Q40_E_ALIGN: return "q40: a pointer or stride is misaligned";
    case Q40_E_WORKSPACE: return "q40: workspace missing or too small";
    case Q40_E_UNSUPPORTED: return "q40: unsupported group size, head dim or index width";
    default: break;
  }
  if (status > 0) return cudaGetErrorString((cudaError_t)status);
  return "q40: unknown status";
}

#ifdef Q40_TRACE
void* q40_trace_ptr = nullptr;
extern "C" void q40_debug_trace(void* buf) { q40_trace_ptr = buf; }
#endif
