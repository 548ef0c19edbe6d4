"""CPU oracle of the PyramidConvBlock hot path: TEST INFRASTRUCTURE, never the product path.

Only tests/, __graft_entry__.smoke() and the CPU-baseline / reference legs of bench.py import this
package.  See oracle.py.
"""
