"""Stands where the reference's build installs its compiled extension (`pshattn*.so`, CMakeLists.txt:69-76)."""
