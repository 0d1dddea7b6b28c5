// Same include path as in the reference tree; the launch_rope / kv_update / flash_attention_* live in gcore/greta_b200.hpp.
#pragma once
#include "gcore/greta_b200.hpp"
