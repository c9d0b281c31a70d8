// Umbrella header of the nt:: host surface over libntb200 (see Tensor.h, functional.h, nn.h).
#pragma once
#include "Tensor.h"
#include "functional.h"
#include "nn.h"
