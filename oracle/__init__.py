"""CPU oracle for the RoDe hot path (test infrastructure, not part of the product).

Only the test-suite, the smoke check and the CPU-baseline leg of the benchmark may import
this package, and only as the checker or the timed baseline.  The shipped package
``rode_b200`` never imports it.

``oracle.cpu``  ctypes front-end of ``rode_oracle.c`` (plain C restatement).
``oracle.ref``  ctypes front-end of the reference's own code compiled into ``oracle/_ref``
                (present only where ``make -C oracle ref`` ran against a reference checkout).
"""
