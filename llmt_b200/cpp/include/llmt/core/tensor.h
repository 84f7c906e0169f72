// llmt's sources include "llmt/core/tensor.h" (its include/llmt/core/tensor.h); here those types live in
// one header, llmt/core/types.h, and this path only forwards to it so that such sources compile
// against this tree unchanged.
#pragma once
#include "llmt/core/types.h"
