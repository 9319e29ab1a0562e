// Shared by the translation units of libevt_b200.so; not part of the C-ABI.
#pragma once
#include <string>

namespace evtb {

// text returned by evtb_last_error() on the calling thread
void set_last_error(const std::string& text);

// number of SMs of the current device (cached per device ordinal); 0 if it cannot be read
int current_device_sm_count();

}  // namespace evtb
