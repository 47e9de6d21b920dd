// Source compatibility: the reference ships types, constants and handles as <rocshmem/rocshmem_common.hpp>
// (include/rocshmem/rocshmem_common.hpp). Programs written against it include this file unchanged.
#pragma once
#include "rocshmem_common.h"
