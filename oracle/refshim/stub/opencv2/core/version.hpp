#pragma once
#define CV_MAJOR_VERSION 4
#define CV_MINOR_VERSION 0
#define CV_VERSION_MAJOR 4
