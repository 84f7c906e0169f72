// Forwarding header: the types live in llmt/core/types.h.
#pragma once
#include "llmt/core/types.h"
