"""Fingerprints of the reference's kernel bodies, by kernel name (written by make_kernel_bodies.py)."""

KNOWN_BODIES: dict[str, frozenset[str]] = {
    # examples/01_vector_add.py:16, benchmarks/bench_dispatch.py:90
    'add_kernel': frozenset({
        '2640a3027fb42c20ef4a640a251e82d04a44a6e26bc4c760322f9dcbbe8d2ef0',
        'fd70fdd794704a4fa5457b8808d7eb8a13723e2a15fbd7de0c774a11ea5be7a8',
    }),
    # examples/08_flash_attention.py:31
    'attention_kernel': frozenset({
        'af23a7ad115c4658044dbcd3cc015289ed97e1fcb94c930b8eceab55e4be4bdb',
    }),
    # examples/10_cumsum.py:18
    'cumsum_kernel': frozenset({
        'fa7ced37faab00ab1267af016e38bb26253fb5f1632887b782264a1c3cb50072',
    }),
    # examples/05_fused_gelu.py:18
    'fused_gelu_kernel': frozenset({
        'f42abff0931ba98eb59b18b6c0d2ede0ec65612a67c497ea01a9f11a7ec120d5',
    }),
    # examples/09_histogram.py:18
    'histogram_kernel': frozenset({
        '0df2ecf02143cdf60db4607939ae6810c4afbfefd4c577bbe2dd1317ae2b34e8',
    }),
    # benchmarks/bench_matmul.py:101
    'int8_matmul_kernel': frozenset({
        '103a94c43e55427ef1fe24a8b387958d93ccc95a490c4fdfec6f61566e327729',
    }),
    # examples/03_layernorm.py:16
    'layernorm_kernel': frozenset({
        'f0f3b9aa16c8077ce2628762adece8c663862e5f95779ff7ebb66c8717397916',
    }),
    # examples/07_matmul_fused.py:18
    'matmul_bias_gelu_kernel': frozenset({
        '17581b0d19114d753e9e9c517b2c2502b99e5814fe04b92358a96d5fc6a699a6',
    }),
    # examples/04_matmul.py:54
    'matmul_desc_kernel': frozenset({
        '1d3dda247222f9f0ca3dcf3851864ee5506d483560861e0df11402eab933fdb3',
    }),
    # examples/04_matmul.py:22
    'matmul_kernel': frozenset({
        '98a41ee1964fd231dd043252e5be20c388994623c9b86e4dae706c94dd94e61d',
    }),
    # examples/06_rmsnorm.py:16
    'rmsnorm_kernel': frozenset({
        '02ec4be9c4042bdc31f03d7cb1efb9550f2d4267f7fe959659c5c7f7724b4ad6',
    }),
    # examples/02_softmax.py:16
    'softmax_kernel': frozenset({
        '191641e6d49792433c8e7b975cfdd5d99f1dfee02b517ce6a4782df61f2133ba',
    }),
}
