// Model weights owned by a context (filled in by the encoder / decoder units).
#include "context.h"

void sb_model_free_internal(sb_ctx* c) { (void)c; }
