"""TEST INFRASTRUCTURE ONLY: CPU oracle for the sparse-embedding hot path.

``oracle.port``   ctypes/numpy front end of the C restatement (``oracle.c``).
``oracle.ref``    loaders for the reference's own compiled host code in
                  ``oracle/_ref`` (built by ``oracle/build_ref.py``).

Only ``tests/``, ``__graft_entry__.smoke()`` and the CPU-baseline legs of
``bench.py`` may import this package.  The product package never does.
"""
