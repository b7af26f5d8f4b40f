"""NVIDIA B200 (Blackwell, sm_100a) hardware model.

Carries every attribute the solver, the cost model and the CLIs read from an arch object
(the set the reference's arch/H100.py:97-119 and arch/H20.py:39-60 define), with B200
values, plus the Blackwell-only parameters of the tcgen05 / TMEM / TMA kernels.
``configure_device`` specialises the model with what the visible device reports, as
H20.configure_device does (arch/H20.py:69-82), but takes a torch device index.
"""

from .Arch import Arch


class B200(Arch):
    def __init__(self, para_opt=True):
        self.para_opt = para_opt
        self.name = "NVIDIA B200"
        self.compute_capability = (10, 0)
        self.global_mem_capacity = "180GB"

        self._set_sm_count(148)
        # Register file and shared memory of one SM.
        self.max_registers_per_sm = 65536
        self.reg_cap = [65536, 255]
        self.smem_cap = [49152]
        self.max_dyn_smem_per_block = 232448  # 227 KB opt-in
        self.shared_mem_config_options = [0, 8, 16, 32, 64, 100, 132, 164, 196, 228]  # KB
        self.max_resident_warps_per_sm = 64
        self.max_resident_blocks_per_sm = 32
        self.smem_bank_size = 4
        self.bank_number = 32

        # Clocks: 1965 MHz boost; long tensor-core loops settle near 1.36 GHz under the 1 kW cap.
        self.sm_clock_hz = 1.965e9
        self.sustained_tensor_clock_hz = 1.36e9
        self.smem_bw_per_sm = 128 * self.sm_clock_hz  # B/s

        # HBM3e: 8 stacks; nominal 8 TB/s (7.7 TB/s on HGX boards); a device-to-device copy
        # measures about 6.5 TB/s read+write.
        self.dram_bw = 8000  # GB/s, the "% of DRAM peak" denominator of the row-wise CLI
        self.dram_bw_measured_copy = 6535.7  # GB/s
        self.dram_latency_s = 1.0e-6
        self.l2_bytes = 126 * 1024 * 1024
        self.l2_bw = 20000  # GB/s, aggregate L2 read bandwidth (order of magnitude, both dies)
        self.bandwidth = [self.dram_bw, self.smem_bw_per_sm * self.sm_nums / 1e9]

        # Compute (GFLOPS).  FP32 CUDA cores: 148 SMs x 128 FMA x 2 x 1.965 GHz.
        self.peak_flops = 148 * 128 * 2 * 1.965
        # Dense fp16/bf16 tensor peak (tcgen05, fp32 accumulation): 2.25 PFLOPS nominal.
        self.peak_tcgen05_flops = 2250000
        self.peak_tc_flops = self.peak_tcgen05_flops
        self.peak_tc_flops_fp32acc = self.peak_tcgen05_flops
        # The CLIs print "% of fp32-acc TC peak" from this attribute (reference:
        # test_gemm_tc.py:157); on B200 the tensor path is tcgen05, so it carries that peak.
        self.peak_mma_sync_flops = self.peak_tcgen05_flops
        self.peak_mma_sync_f16acc_flops = self.peak_tcgen05_flops
        # cuBLAS bf16 8192^3 measured on this class of machine (burst / sustained), GFLOPS.
        self.measured_cublas_flops = 1646900
        self.measured_cublas_flops_sustained = 1399500

        # Blackwell kernel parameters
        self.tmem_columns = 512  # 32-bit columns per SM
        self.tmem_lanes = 128
        self.max_cluster_size = 8
        self.cta_group_sizes = (1, 2)
        self.mma_m_per_cta = (64, 128)  # tcgen05.mma M per CTA
        self.mma_n_max = 256
        self.tma_box_max = 256  # elements per box dimension
        self.swizzle_bytes = (32, 64, 128)
        self.nvlink_bw_gbs = 900  # per direction
        self.num_gpus = 8

        # Optional cost-model knobs the reference exposes on some GPUs.
        self.gemm_excess_stage_penalty = 0.0
        self.fa_cta_sync_penalty = 0.0

    def _set_sm_count(self, sm_nums: int):
        self.sm_nums = sm_nums
        self.compute_max_core = [sm_nums]
        self.mem_max_core = [sm_nums]
        self.compute_sm_partition = [sm_nums, 4]
        self.smem_sm_partition = [sm_nums, 4]

    def configure_device(self, device=0):
        """Fills the device-specific attributes from torch's view of ``device``."""
        import torch

        p = torch.cuda.get_device_properties(device)
        self.name = p.name
        self._set_sm_count(p.multi_processor_count)
        self.global_mem_capacity = f"{p.total_memory / 2**30:.0f}GiB"
        self.l2_bytes = getattr(p, "L2_cache_size", self.l2_bytes)
        self.max_dyn_smem_per_block = getattr(p, "shared_memory_per_block_optin", self.max_dyn_smem_per_block)
        self.bandwidth = [self.dram_bw, self.smem_bw_per_sm * self.sm_nums / 1e9]
        self.num_gpus = torch.cuda.device_count()
        return self
