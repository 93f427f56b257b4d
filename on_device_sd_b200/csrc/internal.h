// Declarations shared between the translation units of libb200moe.so (not part of the ABI).
#pragma once

// Records a message for b200moe_last_error(NULL) in the calling thread and returns `code`.
int b200moe_fail_global(int code, const char* fmt, ...);
