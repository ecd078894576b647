/* flash_train/version.h -- version of the API this build is a drop-in for
 * (reference: include/flash_train/version.h.in:7-10, VERSION.txt = 0.1.0). */
#ifndef FTRAIN_VERSION_H_
#define FTRAIN_VERSION_H_

#define FTRAIN_VERSION_MAJOR 0
#define FTRAIN_VERSION_MINOR 1
#define FTRAIN_VERSION_PATCH 0
#define FTRAIN_VERSION "0.1.0"

#endif
