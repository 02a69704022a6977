"""Every (source, definitions) pair that the library can ask the compiler for with the
head sizes of the shipped configurations; `build()` of the build driver compiles them all."""


def all_variants():
    return [
        ("host_runtime.cpp", ()),
        ("elementwise.cu", ()),
        ("gemm_f32.cu", ()),
        ("attention.cu", ()),
        ("sampling.cu", ()),
        ("attention_decode.cu", ("Q3_HEAD_DIM=128",)),
        ("gemm_skinny_bf16.cu", ()),
        ("attention_prefill.cu", ("Q3_HEAD_DIM=128",)),
        ("attention_decode_static.cu", ("Q3_HEAD_DIM=128",)),
        ("gemm_tcgen05.cu", ()),
        ("attention_prefill_tc.cu", ("Q3_HEAD_DIM=128",)),
    ]
