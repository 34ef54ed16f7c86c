#pragma once
#define PROJECT_VERSION "2.5"
#define GIT_REVISION "unknown"
