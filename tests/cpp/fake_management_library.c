/* Stand-in for the driver's management library in tests: the three entry points libinfinirt looks up, answering
 * with fixed figures (37 % compute, 12 % memory) for any device.  Loaded through INFINIRT_MANAGEMENT_LIBRARY. */
struct utilization {
    unsigned int gpu;
    unsigned int memory;
};

static int fake_device;

int nvmlInit_v2(void) { return 0; }

int nvmlDeviceGetHandleByPciBusId_v2(const char *bus_id, void **device) {
    if (bus_id == 0 || bus_id[0] == '\0') {
        return 2;
    }
    *device = &fake_device;
    return 0;
}

int nvmlDeviceGetUtilizationRates(void *device, struct utilization *out) {
    if (device != &fake_device) {
        return 2;
    }
    out->gpu = 37;
    out->memory = 12;
    return 0;
}
