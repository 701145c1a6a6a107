/* Test infrastructure only.  No-op definitions of the twelve live-viewer entry
 * points the reference declares in src/ncm.h:402-414.  The reference's own
 * src/viewer.c does not compile without SDL2 headers, and nothing on the token
 * loop calls it, so the reference CPU build used as the parity oracle links
 * these stubs instead.  Never linked into the shipped library. */
#include "ncm.h"

int viewer_open(const char *title) { (void)title; return -1; }
void viewer_push(const ViewSnap *s) { (void)s; }
int viewer_stop_requested(void) { return 0; }
void viewer_hold(void) {}
void viewer_close(void) {}
int viewer_active(void) { return 0; }
int viewer_font_test_bmp(const char *path) { (void)path; return -1; }
int viewer_test_frame_bmp(const char *path, int mode) { (void)path; (void)mode; return -1; }
int con_viewer_open(const char *title) { (void)title; return -1; }
void con_viewer_push(const ViewSnap *s) { (void)s; }
void con_viewer_close(void) {}
