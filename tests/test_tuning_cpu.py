"""CPU: the kernel-selection cost model reproduces the measured winners and respects the
tensor-core kernel's shape limits."""
from intrasm_engine_b200.pytorch import tuning


def test_measured_cases():
    # (m, k, n, sparsity) -> winner measured on B200
    cases = [((2048, 512, 128, 0.70), "tensor_core"), ((512, 2048, 128, 0.95), "cuda_core"),
             ((11008, 4096, 64, 0.50), "tensor_core"), ((512, 512, 256, 0.98), "cuda_core")]
    for (m, k, n, sp), want in cases:
        nnz = int(m * k * (1 - sp))
        assert tuning.choose_spmm_kernel(m, k, n, nnz) == want, (m, k, n, sp)


def test_model_against_measured_times():
    assert abs(tuning.tensor_core_us(11008, 4096) - 57.0) < 10     # 49-58 us measured
    assert abs(tuning.tensor_core_us(2048, 512) - 15.0) < 4        # 12.4 us measured
    for (m, nnz, n), measured in (((2048, 315538, 128), 30.8), ((512, 52418, 128), 18.5),
                                  ((512, 25390, 256), 10.3), ((11008, 22544909, 64), 450.0)):
        assert abs(tuning.cuda_core_us(m, nnz, n) - measured) < 0.15 * measured


def test_shape_limits():
    assert not tuning.tensor_core_supported(512, 48, 16, 16)     # n not a multiple of 64
    assert not tuning.tensor_core_supported(512, 320, 16, 16)    # n too large
    assert not tuning.tensor_core_supported(70000, 64, 16, 16)   # 16-bit indices cannot reach
    assert tuning.tensor_core_supported(70000 - 70000 % 8, 64, 16, 32)
    assert tuning.choose_spmm_kernel(512, 512, 48, 100000) == "cuda_core"
    assert tuning.choose_spmm_kernel(512, 512, 64, 100000, value_bits=32) == "cuda_core"


def test_monotone_in_density():
    prev = "cuda_core"
    for sp in (0.99, 0.95, 0.9, 0.8, 0.5, 0.2):
        nnz = int(4096 * 4096 * (1 - sp))
        cur = tuning.choose_spmm_kernel(4096, 4096, 128, nnz)
        assert not (prev == "tensor_core" and cur == "cuda_core")  # once dense enough, stays
        prev = cur
    assert prev == "tensor_core"
