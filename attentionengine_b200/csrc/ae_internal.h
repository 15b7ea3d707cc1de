// Internal (not part of the C ABI): shared between the translation units of libae_b200.so.
#pragma once
// Sets the text that ae_last_error() returns on the calling thread.
void ae_internal_set_error(const char* msg);
