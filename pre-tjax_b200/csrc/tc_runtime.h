// Host-only declarations shared between the tensor-core translation units.
#pragma once
namespace ptj {
namespace tc {
// Device address of the word in which kernels record a run-out wait (current device); nullptr on error.
unsigned int* fault_word();
}  // namespace tc
}  // namespace ptj
