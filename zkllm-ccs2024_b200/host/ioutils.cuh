// Raw binary tensor files (the reference's ioutils.cuh:5-9): no header, the
// element count is the file length divided by the element size.
#pragma once
#include <iostream>
#include <string>
using namespace std;

// file length in bytes
uint findsize(const string& path);
// the first n_bytes of the file -> device buffer
void loadbin(const string& path, void* device_dst, uint n_bytes);
// device buffer -> file (created or truncated)
void savebin(const string& path, const void* device_src, uint n_bytes);
