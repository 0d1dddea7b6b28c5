// Same include path as in the reference tree; the backend classes live in gcore/greta_b200.hpp.
#pragma once
#include "gcore/greta_b200.hpp"
