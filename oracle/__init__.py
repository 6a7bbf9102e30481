"""TEST INFRASTRUCTURE -- checkers for the CUDA kernels, never the product.

``oracle.cpu``  numpy front end of host_ref.cpp (the CPU restatement).
``oracle.ref``  torch front end of ref_shim.cu (the reference's own CUDA kernels).
Only tests/, __graft_entry__.smoke() and bench.py's baseline legs import this.
"""
