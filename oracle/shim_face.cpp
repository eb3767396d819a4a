// TEST INFRASTRUCTURE ONLY: links this repository's drop-in carat::Gemma4BatchModelRunner
// (carat_b200/shim/batch_model_runner_shim.cpp, compiled against the reference's own headers)
// with pointer-table weight arenas and the same extern "C" face the reference's runner gets in
// ref_cuda_shim.cu, so a GPU test can drive the shim exactly as it drives the reference:
// `make -C oracle shim REFERENCE=<carat checkout>` -> _ref/libshim_runner.so, which loads
// ../../carat_b200/libcarat_b200.so.
#include "carat/batch_model_runner.h"
#include "carat/device_weights.h"
#include "carat/gemma4_config.h"

#include <cstring>
#include <map>
#include <memory>
#include <optional>
#include <stdexcept>
#include <string>
#include <vector>

namespace carat {
#include "ref_arenas.inc"
} // namespace carat

#include "ref_face_helpers.inc"

extern "C" {

const char *ref_last_error(void) { return last_error.c_str(); }

#include "ref_runner_face.inc"

} // extern "C"
