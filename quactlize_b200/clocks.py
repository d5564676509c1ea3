"""Read-only sampling of the SM clock and the throttle reasons DURING a timed region (NVML in a thread, nvidia-smi in a
child process when NVML cannot be loaded).  Used by bench.py and by the bench_suite / bench_ep command lines; nothing here
changes a setting of the GPU."""
from __future__ import annotations

import subprocess
import threading
import time

import numpy as np
import torch


class ClockSampler:
    """SM clock and throttle reasons sampled DURING a timed region: NVML in a thread (every 2 ms), or nvidia-smi in a
    child process when NVML cannot be loaded.  Read-only queries."""
    Q = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown," \
        "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"
    BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}
    _nvml = None

    def __init__(self, cuda_index):
        self.index = cuda_index
        self.handle = None
        if ClockSampler._nvml is None:
            try:
                import pynvml
                pynvml.nvmlInit()
                ClockSampler._nvml = pynvml
            except Exception:
                ClockSampler._nvml = False
        if ClockSampler._nvml:
            nv = ClockSampler._nvml
            try:
                uuid = str(torch.cuda.get_device_properties(cuda_index).uuid)
                uuid = uuid if uuid.startswith("GPU-") else "GPU-" + uuid
                self.handle = nv.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                try:
                    self.handle = nv.nvmlDeviceGetHandleByIndex(cuda_index)
                except Exception:
                    self.handle = None

    def start(self):
        self.sm, self.mask, self.mx, self.stop_flag, self.proc, self.rows = [], 0, None, False, None, []
        if self.handle is not None:
            nv = ClockSampler._nvml
            try:
                self.mx = float(nv.nvmlDeviceGetMaxClockInfo(self.handle, nv.NVML_CLOCK_SM))
            except Exception:
                self.mx = None

            def loop():
                while not self.stop_flag:
                    try:
                        self.sm.append(float(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM)))
                        self.mask |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                    except Exception:
                        pass
                    time.sleep(0.002)
            self.thread = threading.Thread(target=loop, daemon=True)
            self.thread.start()
            return self
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "50"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=lambda: [self.rows.append([c.strip() for c in ln.split(",")]) for ln in self.proc.stdout],
                             daemon=True).start()
        except Exception:
            self.proc = None
        return self

    def stop(self):
        if self.handle is not None:
            self.stop_flag = True
            self.thread.join(timeout=1.0)
            reasons = sorted(k for k, b in self.BITS.items() if self.mask & b)
            return {"sm_mhz": float(np.median(self.sm)) if self.sm else None, "sm_max_mhz": self.mx, "reasons": reasons,
                    "samples": len(self.sm), "via": "nvml"}
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no clock source"], "samples": 0}
        time.sleep(0.12)
        self.proc.terminate()
        sm, mx, reasons = [], None, set()
        for r in self.rows:
            try:
                sm.append(float(r[0])); mx = float(r[1])
                for nme, v in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], r[2:6]):
                    if v.lower().startswith("active"):
                        reasons.add(nme)
            except Exception:
                continue
        return {"sm_mhz": float(np.median(sm)) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "via": "nvidia-smi"}
