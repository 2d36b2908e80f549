"""Bounded models of the runtime's concurrency protocols, checked exhaustively by ``utils.model_check.explore``.

* ``tp_exchange``   arrival and ready counters of the tensor-parallel exchange (scatter GEMM -> exchange kernel -> consumer
                    GEMM), cleared by whoever consumed them, over several back-to-back exchanges
* ``stream_k``      the fix-up order of the stream-K GEMM under limited CTA residency

Each model has a configuration that follows the kernels and one that breaks the rule the kernels rely on; the tests
require the first to pass and the second to produce a counterexample.
"""
