// Host-side program table and the compile-time dispatch from a table row to a kernel instance.
#pragma once

#include <cstdint>
#include <type_traits>

#include "fpt_common.h"
#include "fpt_packed.cuh"

namespace fpt {

struct ProgramRow {
    const char* name;
    int dtype, source, shape, degree;
    uint16_t clamp;
    uint16_t c[7];
};

const ProgramRow* program_table(int* count);
// nullptr when the combination does not exist
const ProgramRow* find_program(int function, int direction, int degree, int dtype, int source);

inline ProgramWords program_words(const ProgramRow& r) {
    ProgramWords w;
    w.clamp = uint32_t(r.clamp) * 0x00010001u;
    for (int k = 0; k < 7; ++k) w.c[k] = uint32_t(r.c[k]) * 0x00010001u;
    return w;
}

template <int V>
using IC = std::integral_constant<int, V>;

// Calls f(IC<shape>, IC<degree>) for the row's shape/degree if `MASK` (bit per Shape) allows it.
template <unsigned MASK, class F>
int dispatch_shape_degree(int shape, int degree, F&& f) {
#define FPT_DEG_SWITCH(S)                                  \
    if constexpr ((MASK >> S) & 1u) {                      \
        if (shape == S) {                                  \
            switch (degree) {                              \
            case 3: return f(IC<S>{}, IC<3>{});            \
            case 4: return f(IC<S>{}, IC<4>{});            \
            case 5: return f(IC<S>{}, IC<5>{});            \
            case 6: return f(IC<S>{}, IC<6>{});            \
            default: return FPT_ERR_UNKNOWN_PROGRAM;       \
            }                                              \
        }                                                  \
    }
    FPT_DEG_SWITCH(kOddHalf)
    FPT_DEG_SWITCH(kOdd)
    FPT_DEG_SWITCH(kOddSat)
    FPT_DEG_SWITCH(kSwish)
    FPT_DEG_SWITCH(kXmulHalf)
    FPT_DEG_SWITCH(kEven)
#undef FPT_DEG_SWITCH
    return FPT_ERR_UNSUPPORTED_SHAPE;
}

template <class F>
int dispatch_dtype(int dtype, F&& f) {
    if (dtype == kFp16) return f(IC<kFp16>{});
    if (dtype == kBf16) return f(IC<kBf16>{});
    return FPT_ERR_BAD_ENUM;
}

}  // namespace fpt
