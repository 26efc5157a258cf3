// Same include path as the reference tree; the definitions live in llama_weights.h.
#pragma once
#include "src/weights/llama/llama_weights.h"
