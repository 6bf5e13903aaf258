// Registration hook that lets further binding files add functions to the one extension module.
#pragma once
#include <pybind11/pybind11.h>
void sg_register_extra(pybind11::module_& m);
void sg_register_device_io(pybind11::module_& m);  // device_file_io.cpp
// Adds n to the extension-wide count of kernels launched (read through launch_count()).
void sg_count_launch(int n);
// The device int32 word that kernels set when a bounded wait runs out.
int* sg_error_flag();
