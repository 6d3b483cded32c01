// Internal alias: the kernels implement exactly the raw entry points of the public header.
#pragma once
#include "mycaffe_attn.h"
