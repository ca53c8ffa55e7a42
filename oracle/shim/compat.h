// Force-included (-include) when compiling the unmodified reference sources:
// glibc declares sinf & co. in the global namespace only, the reference calls
// them as std::sinf etc. (src/backend/cpu/arithmetic.cpp:201-274).
#pragma once
#ifdef __cplusplus
#include <cmath>
namespace std {
using ::sinf; using ::cosf; using ::tanf; using ::expf; using ::sqrtf;
using ::logf; using ::powf; using ::tanhf; using ::fabsf;
}
#endif
