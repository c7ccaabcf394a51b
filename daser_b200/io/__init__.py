"""Storage engine binding: cuFile, io_uring and POSIX back ends behind one asynchronous interface."""
