// Stand-in for the Windows <io.h> that the reference's llama2 headers include.
// Used only to compile the reference's own llama2_cpu.cpp, in place, as a test checker.
#pragma once
#include <unistd.h>
#include <fcntl.h>
#include <sys/mman.h>
#include <sys/types.h>
