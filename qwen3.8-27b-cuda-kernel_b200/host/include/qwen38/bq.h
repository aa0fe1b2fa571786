// Source-compatibility header: the declarations of the reference's include/qwen38/bq.h live in
// qwen38/api.h together with the rest of the host API.
#pragma once
#include "qwen38/api.h"
