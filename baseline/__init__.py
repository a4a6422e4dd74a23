"""Reference-side legs: the install recipe for the reference package
(install_reference.sh -> baseline/_ref/, git-ignored), the worker that runs the
reference's own packer and Triton kernels in a process of its own
(reference_worker.py) and the seeded workloads both sides generate
(workloads.py).  Nothing here is on the product path."""
