"""CPU oracle of the decode path — TEST INFRASTRUCTURE, not product code.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline /
reference arm may import this package; the product (``machete_b200``) never
does and has no CPU fallback.
"""

from .decode_oracle import *  # noqa: F401,F403
