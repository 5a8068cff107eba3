"""Every public name of the reference's crate root resolves from the package root."""
import rust_neural_network_b200 as rn


def test_every_root_export_resolves():
    missing = []
    for name in rn.__all__:
        try:
            getattr(rn, name)
        except Exception as e:          # noqa: BLE001
            missing.append((name, repr(e)))
    assert not missing, missing
    assert rn.VERSION.startswith("2.1.0")
    assert rn.blas_matmul is rn.blas.matmul and rn.LinearAttentionLayer.elu(64).scale == 0.125
    assert rn.KernelKind.Relu2.to_u8() == 1 and rn.AttentionKind is rn.looped_transformer.AttentionKind
    assert rn.NativeBackend().name().startswith("native") and "tcgen05" in rn.NVIDIA_PTX_KERNEL
    assert rn.nn.NormalMoE is rn.NormalMoE
