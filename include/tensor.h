// Forwarding header: small-llm code that includes "tensor.h" finds the same names in small_llm.hpp.
#pragma once
#include "small_llm.hpp"
