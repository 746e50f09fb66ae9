/* Minimal NVML stand-in: the reference's post-cuInit hook resolves and calls
 * these five entry points unconditionally.  Zero devices, no processes. */
typedef int nvmlReturn_t;
nvmlReturn_t nvmlInit_v2(void) { return 0; }
nvmlReturn_t nvmlDeviceGetCount_v2(unsigned int *count) { *count = 0; return 0; }
nvmlReturn_t nvmlDeviceGetHandleByIndex_v2(unsigned int index, void **device) { (void)index; *device = 0; return 0; }
nvmlReturn_t nvmlDeviceGetGraphicsRunningProcesses_v3(void *d, unsigned int *n, void *infos) { (void)d; (void)infos; *n = 0; return 0; }
nvmlReturn_t nvmlDeviceGetComputeRunningProcesses_v3(void *d, unsigned int *n, void *infos) { (void)d; (void)infos; *n = 0; return 0; }
