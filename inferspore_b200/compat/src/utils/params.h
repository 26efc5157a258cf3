// Name -> scalar dictionaries used to bundle launch arguments
// (reference: src/utils/params.h).
#pragma once
#include <string>
#include <unordered_map>

using IntDict = std::unordered_map<std::string, int>;
using floatDict = std::unordered_map<std::string, float>;
