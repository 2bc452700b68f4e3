// Same include path as the reference's uocr/continuous_batch.h; everything lives in rswa_host.h.
#pragma once
#include "uocr/rswa_host.h"
