// Test infrastructure: see faiss/gpu/StandardGpuResources.h in this directory.
#pragma once
