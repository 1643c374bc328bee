// Raw binary tensor files (the reference's ioutils.cuh:5-9): no header, the
// element count is the file length divided by the element size.
#pragma once
#include <iostream>
#include <string>
using namespace std;

// device buffer -> file
void savebin(const string& filename, const void* gpudata, uint size);
// file length in bytes
uint findsize(const string& filename);
// file -> device buffer
void loadbin(const string& filename, void* gpudata, uint size);
