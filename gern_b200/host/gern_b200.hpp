// Umbrella header of the C++ host layer above the C ABI.
#pragma once
#include "annotations.hpp"
#include "compose.hpp"
#include "impl.hpp"
#include "runner.hpp"
