// Stand-in declarations for the uGDS storage library, which the reference
// executor includes (src/kimi_exec.cu:22) but which is an empty, un-vendored
// submodule in the reference checkout.  Only the names the reference's source
// mentions are declared, shaped after their call sites (src/kimi_exec.cu:56-66,
// :105-110, :130, :219-235, :616-618).  Every function reports failure: the
// pinning harness launches the reference's kernels directly and never touches
// the storage layer.
#pragma once
#include <sys/types.h>
#include <cstddef>

typedef struct uGDSHandleOpaque *uGDSHandle_t;
enum { UGDS_SUCCESS = 0, UGDS_STUB_ERROR = 1 };
enum { UGDS_HANDLE_TYPE_OPAQUE_FD = 1 };
struct uGDSError_t { int err; };
struct uGDSDescr_t {
  int type;
  union { int fd; void *ptr; } handle;
};

inline const char *uGDS_status_error(int) { return "uGDS is not present (stub)"; }
inline uGDSError_t uGDSDriverOpen() { return {UGDS_STUB_ERROR}; }
inline uGDSError_t uGDSDriverClose() { return {UGDS_STUB_ERROR}; }
inline uGDSError_t uGDSHandleRegister(uGDSHandle_t *, uGDSDescr_t *) { return {UGDS_STUB_ERROR}; }
inline void uGDSHandleDeregister(uGDSHandle_t) {}
inline uGDSError_t uGDSBufRegister(const void *, size_t, int) { return {UGDS_STUB_ERROR}; }
inline uGDSError_t uGDSBufDeregister(const void *) { return {UGDS_STUB_ERROR}; }
inline ssize_t uGDSRead(uGDSHandle_t, void *, size_t, off_t, off_t) { return -1; }
inline ssize_t uGDSWrite(uGDSHandle_t, const void *, size_t, off_t, off_t) { return -1; }
