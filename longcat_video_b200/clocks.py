"""Clock and throttle-reason sampling for the benchmark (reads nvidia-smi; changes nothing)."""
import statistics
import subprocess
import threading
import time


class ClockSampler:
    """Samples nvidia-smi clocks / throttle reasons while the timed region runs.

    nvidia-smi needs a moment to start, so ``start()`` is called well before the timed region (before the warm-up);
    ``mark_begin()`` / ``mark_end()`` bracket the timed region and ``stop()`` summarises the samples that fell inside
    it (all samples taken under load if the region was shorter than one sampling period)."""
    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None
        self.t_begin = self.t_end = None

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.Q}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._read, daemon=True).start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), [c.strip() for c in line.split(",")]))

    def mark_begin(self):
        self.t_begin = time.time()

    def mark_end(self):
        self.t_end = time.time()

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.1)
        self.proc.terminate()

        def summarise(rows):
            sm, mx, reasons = [], None, set()
            for _, r in rows:
                try:
                    sm.append(float(r[0]))
                    mx = float(r[1])
                except (ValueError, IndexError):
                    continue
                for name, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[3:7]):
                    if v.lower().startswith("active"):
                        reasons.add(name)
            return sm, mx, reasons

        inside = self.rows
        if self.t_begin is not None and self.t_end is not None:
            inside = [x for x in self.rows if self.t_begin <= x[0] <= self.t_end + 0.03]
        sm, mx, reasons = summarise(inside)
        window = "timed region"
        if not sm:  # the region was shorter than a sampling period: fall back to every sample taken under load
            sm, mx, reasons = summarise(self.rows)
            window = "whole run (timed region shorter than a sampling period)"
        busy = [x for x in sm if mx and x > 0.5 * mx] or sm
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": mx, "reasons": sorted(reasons),
                "samples": len(sm), "window": window}
