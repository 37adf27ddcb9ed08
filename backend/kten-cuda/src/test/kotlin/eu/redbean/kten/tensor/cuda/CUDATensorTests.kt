package eu.redbean.kten.tensor.cuda

import eu.redbean.kten.api.tensor.operations.TensorOperations
import eu.redbean.kten.api.tensor.operations.TensorOperationsGarbageCollector
import eu.redbean.kten.api.tensor.platform.DeviceType
import eu.redbean.kten.api.tensor.platform.PlatformProvider
import eu.redbean.kten.api.tensor.store.AbstractRawTensor
import eu.redbean.kten.tensor.tests.TensorTestsBase
import org.junit.jupiter.api.AfterEach
import org.junit.jupiter.api.BeforeAll
import org.junit.jupiter.api.BeforeEach
import org.junit.jupiter.api.TestInstance

/**
 * kten's backend-agnostic suite on the CUDA platform, one GC scope per test (the pattern of
 * backend/kten-opencl/src/test/.../OpenCLTensorTests.kt).  Tests that use operations outside the
 * float32 hot path fail with UnsupportedOperationException until those operations are added.
 */
@TestInstance(TestInstance.Lifecycle.PER_CLASS)
class CUDATensorTests : TensorTestsBase() {

    private lateinit var gc: TensorOperationsGarbageCollector
    private lateinit var platformKey: String

    @BeforeAll
    @Suppress("UNCHECKED_CAST")
    fun setupDefaultOps() {
        val info = PlatformProvider.findPlatform { it.platformImplementationType == "CUDA" && it.deviceType == DeviceType.GPU }
        platformKey = info.platformKey
        PlatformProvider.registerAsDefault(platformKey, PlatformProvider.tensorOperations(platformKey) as TensorOperations<AbstractRawTensor<Any>>, info)
    }

    @BeforeEach
    fun setupGc() {
        gc = PlatformProvider.tensorOperations(platformKey).garbageCollector()
    }

    @AfterEach
    fun tearDownGc() = gc.close()
}
