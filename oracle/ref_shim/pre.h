// Force-included before the reference's llama2_cpu.cpp: the handful of Windows
// names that file uses (LONG, two Win32 error codes, _open/_close).
#pragma once
#include <stdint.h>
#include <stddef.h>
typedef long LONG;
#ifndef ERROR_OUTOFMEMORY
#define ERROR_OUTOFMEMORY 14
#endif
#ifndef ERROR_FILE_INVALID
#define ERROR_FILE_INVALID 1006
#endif
#define _open open
#define _close close
