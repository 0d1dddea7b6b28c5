// Same include path as in the reference tree; the launch_rmsnorm_naive / add / silu / mul / embedding / argmax live in gcore/greta_b200.hpp.
#pragma once
#include "gcore/greta_b200.hpp"
