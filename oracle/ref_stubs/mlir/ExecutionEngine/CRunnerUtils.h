// Empty stand-in: conv-validation-wrappers.cpp includes this header but uses nothing from it.
#pragma once
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <ctime>
#include <limits>
