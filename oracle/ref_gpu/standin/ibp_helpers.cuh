// Empty stand-in.  The reference's comp_cache/static_cache.cuh includes a header of this name from a
// compression library that is not part of its tree; the operator kernels that ref_ops_driver.cu runs
// (batch_generate, counter_update, construct_graph, ClearPosMap) use nothing of it.  Only the build of
// that one driver puts this directory on its include path.
#pragma once
