// Stand-in for the header the reference's CMake build generates from src/TackerConfig.h.in (version numbers, log
// path, build type): the ori_kernel sources include it through Logger.h.  Test infrastructure only.
#pragma once
#define Tacker_VERSION_MAJOR 0
#define Tacker_VERSION_MINOR 0
#define Tacker_VERSION_PATCH 0
#define LOG_FILE_PATH "/dev/null"
#define COMPILE_TIMESTAMP ""
#define CMAKELISTS_PATH "."
#define BUILD_TYPE "RELEASE"
