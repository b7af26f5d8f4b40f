"""Base class of the hardware models (same accessors as the reference's arch/Arch.py:1-43)."""

import math


class Arch:
    para_opt = True

    def memory_bw(self, mem_level, num_core=-1):
        bw = self.bandwidth[mem_level]
        return bw if num_core == -1 else bw * self._memory_penalty(num_core)

    def _peak_flops(self, num_core=-1):
        return self.peak_flops if num_core == -1 else self.peak_flops * self._compute_penalty(num_core)

    def _reg_cap(self, mem_level):
        return self.reg_cap[mem_level]

    def mem_cap(self, mem_level):
        return self.smem_cap[mem_level]

    @staticmethod
    def _penalty(max_cores, num_core):
        worst = 1.0
        for mx, real in zip(max_cores, num_core):
            if real is not None:
                worst = min(worst, 1.0 / math.ceil(real / mx) / (mx / real))
        return worst

    def _memory_penalty(self, num_core):
        return self._penalty(self.mem_max_core, num_core) if self.para_opt else 1

    def _compute_penalty(self, num_core):
        return self._penalty(self.compute_max_core, num_core) if self.para_opt else 1

    def _smem_bank_size(self):
        return self.smem_bank_size

    def _bank_number(self):
        return self.bank_number
