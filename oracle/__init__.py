"""CPU oracle of the decode path.  Test infrastructure: imported only by tests/, by
``__graft_entry__.smoke()`` and by the CPU-baseline / ``--impl reference`` legs of bench.py."""
