// Test infrastructure: see StandardGpuResources.h in this directory.
#pragma once
#include "StandardGpuResources.h"
