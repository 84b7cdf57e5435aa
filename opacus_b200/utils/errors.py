"""Exceptions raised by the native layer."""


class CommTimeoutError(RuntimeError):
    """A kernel gave up on a bounded wait (a peer's flag, a copy in flight, a pipeline barrier).

    Every device-side wait of this package is limited to about two seconds; on expiry the kernel records
    which wait it was in a host-visible status block, unwinds and returns, and the next call into the
    native module raises this error.  The CUDA context stays usable; the results of the step that timed
    out are invalid.  In a multi-GPU job it usually means that a peer rank died or never reached the
    matching call: restart from the last checkpoint.
    """
