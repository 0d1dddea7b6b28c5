// Same include path as in the reference tree; the launch_gemm_* entry points live in gcore/greta_b200.hpp.
#pragma once
#include "gcore/greta_b200.hpp"
