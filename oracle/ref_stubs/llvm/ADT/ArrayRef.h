// Empty stand-in: conv-validation-wrappers.cpp includes this header but uses nothing from it.
#pragma once
