// Status codes that the C launchers return (0 = launched).
#pragma once
#define LSE_OK 0
#define LSE_BAD_ARGUMENT 1
#define LSE_LAUNCH_FAILED 2
