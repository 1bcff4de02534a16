// Exception hierarchy and check macros shared by every native component.
//
// Parity: the reference throws MCCLError and five subclasses from a
// DISTRO_CHECK macro that prefixes file:line (csrc/common/Errors.hpp:9-66).
// This build keeps the same class names (Python maps them to RuntimeError /
// TimeoutError) and adds CudaError for runtime-API and driver-API failures.
#pragma once

#include <sstream>
#include <stdexcept>
#include <string>

namespace mccl {

class MCCLError : public std::runtime_error {
 public:
  explicit MCCLError(const std::string& what) : std::runtime_error(what) {}
};

#define MCCL_DEFINE_ERROR(Name)                                   \
  class Name : public MCCLError {                                 \
   public:                                                        \
    explicit Name(const std::string& what) : MCCLError(what) {}   \
  }

MCCL_DEFINE_ERROR(TransportError);  // socket / peer-mapping failures
MCCL_DEFINE_ERROR(CudaError);       // cudaError_t / CUresult failures
MCCL_DEFINE_ERROR(TensorError);     // bad device, dtype, layout or shape
MCCL_DEFINE_ERROR(TimeoutError);    // a bounded wait ran out (host or device)
MCCL_DEFINE_ERROR(ProtocolError);   // wire-format or ordering violation
#undef MCCL_DEFINE_ERROR

namespace detail {
inline std::string located(const char* file, int line, const std::string& msg) {
  std::ostringstream os;
  const char* base = file;
  for (const char* p = file; *p; ++p)
    if (*p == '/') base = p + 1;
  os << "[mccl " << base << ":" << line << "] " << msg;
  return os.str();
}
}  // namespace detail

}  // namespace mccl

// Throws ErrType with a located message when cond is false.  The message
// argument is a stream expression: MCCL_CHECK_T(x > 0, TensorError, "x=" << x).
#define MCCL_CHECK_T(cond, ErrType, streamexpr)                               \
  do {                                                                        \
    if (!(cond)) {                                                            \
      std::ostringstream _mccl_os;                                            \
      _mccl_os << streamexpr;                                                 \
      throw ::mccl::ErrType(                                                  \
          ::mccl::detail::located(__FILE__, __LINE__, _mccl_os.str()));       \
    }                                                                         \
  } while (0)

#define MCCL_CHECK(cond, streamexpr) MCCL_CHECK_T(cond, MCCLError, streamexpr)
#define MCCL_CHECK_TENSOR(cond, streamexpr) MCCL_CHECK_T(cond, TensorError, streamexpr)

// Old spelling kept so code written against the reference macro names builds.
#define DISTRO_CHECK(cond, msg) MCCL_CHECK(cond, msg)
#define DISTRO_CHECK_TENSOR(cond, msg) MCCL_CHECK_TENSOR(cond, msg)
