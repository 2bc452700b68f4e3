// Same include path as the reference's uocr/memory_pool.h; everything lives in rswa_host.h.
#pragma once
#include "uocr/rswa_host.h"
