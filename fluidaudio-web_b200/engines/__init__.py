"""Engine forwards written only against ComputeContext members (the reference's rule,
docs/ARCHITECTURE.md:31-38): the same functions run on CudaContext and on any other backend
object with the same methods."""
