// Forwarding header: the whole quantized-inference API lives in forge_b200.hpp.
#pragma once
#include "../../forge_b200.hpp"
