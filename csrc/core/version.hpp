// Version constants exported to Python as _C.__version__ and
// _C.__protocol_version__ (the reference's tests look for both on the
// extension module: tests/test_build.py:43-46; values from
// csrc/common/Version.hpp:3-9).
#pragma once

#define MCCL_VERSION_MAJOR 0
#define MCCL_VERSION_MINOR 4
#define MCCL_VERSION_PATCH 0
#define MCCL_VERSION_STRING "0.4.0"
// Version of the framed TCP protocol (handshake + send/recv headers).
#define MCCL_PROTOCOL_VERSION 1
