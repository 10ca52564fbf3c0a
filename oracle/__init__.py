"""TEST INFRASTRUCTURE: CPU oracle of the Roller hot path (search restatement, fp64/fp32 GEMM
references, plain-C kernel-arithmetic models). Imported only by tests/, the smoke check and
bench.py's CPU-baseline / reference arm -- never by the product package."""
