#pragma once
#include <cstdint>
namespace llmt::kernels {
// Which score entries are valid (llmt mask.h): Causal = query q sees keys <= q.
enum class MaskKind : uint8_t { None, Causal };
struct MaskSpec {
    MaskKind kind = MaskKind::None;
};
}  // namespace llmt::kernels
